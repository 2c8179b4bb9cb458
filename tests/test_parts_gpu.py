"""Each part alone against the plain implementation; the run order as data (a layer named twice, a
layer reading another layer's cache); a toy mixer with state of its own, a toy feed-forward and a toy
position encoding registered from this file and built and stepped without a change to the framework;
and greedy / sampled generation through the entry point."""

import subprocess
import sys
from pathlib import Path

import pytest
import torch

from tests import helpers as H
from tests.conftest import TINY
from tests.plain import minimax_m3_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = Path(__file__).resolve().parent.parent


def _ctx(T, pos=None, req=None, dtype=torch.float32, n_axes=1):
    from quanta_b200 import kernels
    from quanta_b200.parts.base import StepContext
    pos = torch.arange(T, dtype=torch.int32) if pos is None else pos
    req = torch.zeros(T, dtype=torch.int32) if req is None else req
    positions = pos.view(T, 1).repeat(1, n_axes).contiguous()      # a text token feeds its position to every axis
    return StepContext(n_tokens=T, positions=positions.to(DEV), tok_pos=pos.to(DEV), tok_req=req.to(DEV),
                       req_slot=torch.zeros(1, dtype=torch.int32, device=DEV),
                       req_start=torch.tensor([0, T], dtype=torch.int32, device=DEV),
                       req_len_after=torch.tensor([T], dtype=torch.int32, device=DEV),
                       status=kernels.new_status(DEV), dtype=dtype, max_new_tokens_per_req=T, max_len_after=T)


def _loaded(model_dirs, name, dtype="float32"):
    from quanta_b200.engine.model import load_model
    return load_model(model_dirs[name], dtype=dtype)[0]


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_norm_attention_experts_alone(model_dirs, plain_models, name):
    from quanta_b200.parts.base import LayerCache
    model = _loaded(model_dirs, name)
    weights, cfg = plain_models[name]
    blk = model.blocks[1]
    T, Hd = 21, cfg["H"]
    torch.manual_seed(0)
    x = torch.randn(T, Hd)
    ctx = _ctx(T, n_axes=blk.mixer.position.n_axes)
    p = "model.layers.1."
    # norm
    h = x.clone().to(DEV)
    out = torch.empty(T, Hd, device=DEV)
    blk.mixer_norm.forward(h, None, out)
    assert torch.allclose(out.cpu(), P.rms_norm(x, weights[p + "input_layernorm.weight"], cfg["eps"]), atol=1e-5)
    # mixer: whole sequence through the paged cache
    page = 4
    n_pages = -(-T // page)
    spec = blk.mixer.cache_spec()
    kc = torch.zeros(n_pages, spec.streams[0].heads, page, spec.streams[0].width, device=DEV)
    cache = LayerCache(kc, torch.zeros_like(kc), page, torch.arange(n_pages, dtype=torch.int32, device=DEV).view(1, -1))
    got = blk.mixer.forward(x.to(DEV), ctx, cache, {})
    W = lambda n: weights[p + "self_attn." + n].float()     # noqa: E731
    q = (x @ W("q_proj.weight").T).reshape(T, cfg["nq"], cfg["hd"])
    k = (x @ W("k_proj.weight").T).reshape(T, cfg["nkv"], cfg["hd"])
    v = (x @ W("v_proj.weight").T).reshape(T, cfg["nkv"], cfg["hd"])
    if cfg["qk_norm"]:
        q = P.qk_norm(q, W("q_norm.weight"), cfg["nq"], cfg["hd"], cfg["qk_norm_type"], cfg["eps"])
        k = P.qk_norm(k, W("k_norm.weight"), cfg["nkv"], cfg["hd"], cfg["qk_norm_type"], cfg["eps"])
    pos = torch.arange(T)
    q, k = P.partial_rope(q, pos, cfg["rd"], cfg["theta"]), P.partial_rope(k, pos, cfg["rd"], cfg["theta"])
    want = P.causal_attention(q, k, v, None, torch.float32) @ W("o_proj.weight").T
    assert torch.allclose(got.cpu(), want, atol=2e-5)
    # feed-forward: router alone, then the whole part (summed over its k slots)
    ffn = blk.feed_forward
    m = p + "block_sparse_moe."
    bias = weights[m + "e_score_correction_bias"] if cfg["bias"] else None
    idx, w = ffn.route(x.to(DEV))
    widx, ww = P.router(x, weights[m + "gate.weight"], bias, cfg["k"], cfg["renorm"], cfg["scale"])
    assert torch.equal(idx.cpu().long(), widx) and torch.allclose(w.cpu(), ww, atol=1e-6)
    y = ffn.forward(x.to(DEV), ctx)
    experts = [tuple(weights[f"{m}experts.{e}.{n}.weight"] for n in ("w1", "w3", "w2")) for e in range(cfg["E"])]
    want = P.moe(x, weights[m + "gate.weight"], bias, experts, cfg["k"], cfg["renorm"], cfg["scale"], None, torch.float32)
    assert y.shape == (T, cfg["k"], Hd)
    assert torch.allclose(y.sum(1).cpu(), want, atol=2e-5)
    assert int(ctx.status[0]) == 0


def test_rotary_part_with_sections_equals_the_plain_ladder():
    from quanta_b200.parts.rotary import PartialRotary
    plain_ = PartialRotary(48, 24, 25000.0)
    sect = PartialRotary(48, 24, 25000.0, sections=[4, 4, 4])
    inv, axis, rd, n_axes = sect.rotary_tables(DEV)
    assert n_axes == 3 and axis.tolist() == [0] * 4 + [1] * 4 + [2] * 4 and rd == 24
    assert torch.equal(inv.cpu(), P.rope_inv_freq(24, 25000.0)) and torch.equal(inv, plain_.rotary_tables(DEV)[0])
    with pytest.raises(ValueError, match="sum"):
        PartialRotary(48, 24, 1e4, sections=[4, 4])


def test_a_dense_feed_forward_from_the_frameworks_kernels():
    """A dense SwiGLU is no part of this architecture; as a toy defined here it shows a feed-forward built
    from the library product and the fused activation kernel."""
    from quanta_b200 import kernels
    from quanta_b200.matmul import empty_rows, linear
    from quanta_b200.parts.base import FeedForward, TensorSpec, make, register

    @register("feed_forward", "toy_dense_swiglu")
    class DenseSwiGLU(FeedForward):
        graph_safe = True

        def __init__(self, hidden_size, inner_size, names):
            self.H, self.I, self.names = hidden_size, inner_size, names

        def tensor_specs(self):
            n = self.names
            return [TensorSpec(n["gate"], (self.I, self.H)), TensorSpec(n["up"], (self.I, self.H)),
                    TensorSpec(n["down"], (self.H, self.I))]

        def load(self, fetch):
            self.w_gu = torch.cat([fetch(self.names["gate"]), fetch(self.names["up"])])
            self.w_down = fetch(self.names["down"])

        def forward(self, x, ctx):
            gu = linear(x, self.w_gu)
            act = empty_rows(x.shape[0], self.I, dtype=x.dtype, device=x.device)
            kernels.silu_mul(gu, act)
            return linear(act, self.w_down)

    torch.manual_seed(1)
    Hd, I, T = 72, 100, 9
    ws = {"g": 0.1 * torch.randn(I, Hd), "u": 0.1 * torch.randn(I, Hd), "d": 0.1 * torch.randn(Hd, I)}
    part = make("feed_forward", ("toy_dense_swiglu", dict(hidden_size=Hd, inner_size=I, names={"gate": "g", "up": "u", "down": "d"})))
    part.load(lambda n: ws[n].to(DEV))
    x = torch.randn(T, Hd)
    got = part.forward(x.to(DEV), _ctx(T))
    assert torch.allclose(got.cpu(), P.expert_swiglu(x, ws["g"], ws["u"], ws["d"], None, torch.float32), atol=1e-5)


def _spec_with_schedule(name, schedule):
    from quanta_b200.config import MiniMaxM3Config, resolve
    raw = TINY[name]
    spec = resolve(raw).build_spec(MiniMaxM3Config.from_dict(raw))
    spec.schedule = schedule
    spec.__post_init__()
    return spec


def test_run_order_is_data_a_layer_twice(model_dirs, plain_models):
    """Schedule [0, 1, 0]: layer 0's weights run twice, each run with a cache of its own."""
    from quanta_b200.engine.model import Model
    from quanta_b200.engine.step import Engine
    from quanta_b200.parts.spec import ScheduleEntry
    from quanta_b200.weights import FolderSource
    spec = _spec_with_schedule("A", [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)])
    model = Model(spec, dtype="float32").load(FolderSource(model_dirs["A"]))
    eng = Engine(model, num_pages=32, page_size=4, max_requests=4)
    assert len(eng.kv) == 3
    reqs = {"a": H.random_tokens(29, 512, 1), "b": H.random_tokens(18, 512, 2)}
    want = H.plain_logits(plain_models["A"], reqs, schedule=[0, 1, 0])
    for cut in (H.cut_whole(reqs), H.cut_portions(reqs), H.cut_mixed(reqs, 2, seed=1)):
        got = H.replay(eng, cut)
        assert H.first_wrong(got, want, 2e-5) is None


def test_a_layer_reads_another_layers_cache(model_dirs, plain_models):
    """Schedule entry 2 runs layer 1's weights on the K/V that entry 0 wrote (it writes none): against the
    plain implementation in the same form, under three cuttings."""
    from quanta_b200.engine.model import Model
    from quanta_b200.engine.step import Engine
    from quanta_b200.parts.spec import ScheduleEntry
    from quanta_b200.weights import FolderSource
    spec = _spec_with_schedule("A", [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1, read_cache_of=0)])
    model = Model(spec, dtype="float32").load(FolderSource(model_dirs["A"]))
    eng = Engine(model, num_pages=32, page_size=4, max_requests=4)
    assert sorted(eng.kv) == [0, 1]
    reqs = {"a": H.random_tokens(27, 512, 3), "b": H.random_tokens(40, 512, 4)}
    want = H.plain_logits(plain_models["A"], reqs, schedule=[0, 1, 1], reads_cache_of={2: 0})
    unshared = H.plain_logits(plain_models["A"], reqs, schedule=[0, 1, 1])
    assert float((want[("a", 26)] - unshared[("a", 26)]).abs().max()) > 1e-3          # the shared cache matters
    for cut in (H.cut_whole(reqs), H.cut_tail_decode(reqs, 10), H.cut_portions(reqs), H.cut_mixed(reqs, 2, seed=3)):
        got = H.replay(eng, cut)
        assert H.first_wrong(got, want, 2e-5) is None, H.worst_error(got, want)
    with pytest.raises(ValueError, match="does not run before"):
        _spec_with_schedule("A", [ScheduleEntry(0, read_cache_of=1), ScheduleEntry(1)])


@pytest.mark.parametrize("name,dtype,windows,page_size", [("A", "float32", {1: 9}, 4), ("B", "float32", {0: 21, 2: 6}, 8),
                                                          ("B", "bfloat16", {0: 21, 2: 6}, 8)])
def test_windowed_layers_have_pages_of_their_own(model_dirs, plain_models, name, dtype, windows, page_size):
    """Some layers read a window of keys only: they form cache groups of their own, whose pages go back
    to the pool as the window passes them, while the other layers keep every key."""
    from quanta_b200.config import MiniMaxM3Config, resolve
    from quanta_b200.engine.model import Model
    from quanta_b200.engine.step import Engine
    from quanta_b200.weights import FolderSource
    raw = TINY[name]
    spec = resolve(raw).build_spec(MiniMaxM3Config.from_dict(raw))
    for layer, w in windows.items():
        spec.layers[layer][1]["mixer"][1]["window"] = w
    model = Model(spec, dtype=dtype).load(FolderSource(model_dirs[name]))
    vocab = raw["vocab_size"]
    reqs = {"a": H.random_tokens(90, vocab, 11), "b": H.random_tokens(57, vocab, 12), "c": H.random_tokens(75, vocab, 13)}
    act = None if dtype == "float32" else torch.bfloat16
    want = H.plain_logits(plain_models[name], reqs, act=act, windows=windows)
    if dtype == "float32":
        tol = 2e-5
    else:
        exact = H.plain_logits(plain_models[name], reqs, windows=windows)
        tol = 2.0 * max(float((want[k] - exact[k]).abs().max()) for k in want)
    # the windows matter: without them the logits differ
    full = H.plain_logits(plain_models[name], {"a": reqs["a"]})
    assert float((full[("a", 89)] - want[("a", 89)]).abs().max()) > 100 * tol or dtype != "float32"
    cuts = {"whole": H.cut_whole(reqs), "tail": H.cut_tail_decode(reqs, 32), "portions": H.cut_portions(reqs),
            "mixed": H.cut_mixed(reqs, 3, seed=5)}
    for what, cut in cuts.items():
        eng = Engine(model, num_pages=H.tokens_in_flight(cut, page_size) // page_size, page_size=page_size, max_requests=4)
        groups = eng.manager.stats()["groups"]
        assert sorted(str(g["window"]) for g in groups) == sorted(["None"] + [str(w) for w in set(windows.values())])
        got = H.replay(eng, cut)
        eng.manager.check_invariants()
        bad = H.first_wrong(got, want, tol)
        assert bad is None, (what, bad, H.worst_error(got, want), tol)
        groups = eng.manager.stats()["groups"]
        everything = max(g["high_water"] for g in groups if g["window"] is None)
        for g in groups:
            if g["window"] is not None and what != "whole":
                assert g["high_water"] < everything, "the windowed group gave no page back while it ran"


# ---- toy parts, defined here, registered, built and stepped --------------------------------------------
def _register_toys():
    from quanta_b200.parts.base import FeedForward, Mixer, PositionEncoding, TensorSpec, register

    @register("mixer", "toy_running_mean")
    class RunningMean(Mixer):
        """Output = (decayed running sum of the projected inputs of this request so far) ; the sum and a
        count live in the request's state slot, so portions must carry them across steps."""

        def __init__(self, hidden_size, weight_name, decay):
            self.H, self.weight_name, self.decay = hidden_size, weight_name, decay
            self.w = None

        def tensor_specs(self):
            return [TensorSpec(self.weight_name, (self.H, self.H))]

        def load(self, fetch):
            self.w = fetch(self.weight_name)

        def state_spec(self):
            return {"sum": ((self.H,), torch.float32), "count": ((1,), torch.float32)}

        def forward(self, x, ctx, cache, state):
            proj = (x.float() @ self.w.float().T)
            out = torch.empty_like(proj)
            starts, slots = ctx.host["req_start"], ctx.host["req_slot"]
            for r, slot in enumerate(slots):                     # a toy: plain torch, one request at a time
                s = state["sum"][slot]
                for t in range(starts[r], starts[r + 1]):
                    s.mul_(self.decay).add_(proj[t])
                    state["count"][slot] += 1
                    out[t] = s / state["count"][slot]
            return out.to(x.dtype)

    @register("feed_forward", "toy_two_way_routing")
    class TwoWay(FeedForward):
        """Routes each token to one of two scalings by the sign of its first feature."""

        def __init__(self, hidden_size, scales):
            self.scales = scales

        def forward(self, x, ctx):
            pick = (x[:, :1] > 0).to(x.dtype)
            return x * (pick * self.scales[0] + (1 - pick) * self.scales[1])

    @register("position", "toy_linear_ladder")
    class LinearLadder(PositionEncoding):
        """Another position encoding: frequencies fall linearly instead of geometrically."""

        def __init__(self, rotary_dim):
            self.rd = rotary_dim

        def rotary_tables(self, device):
            inv = (1.0 - torch.arange(self.rd // 2, dtype=torch.float32) / (self.rd // 2)).to(device)
            return inv, None, self.rd, 1


def _toy_plain(ws, ids, decay, scales, eps):
    """Whole-sequence plain version of the toy model: embedding, [norm, running mean, norm, two-way] x 2."""
    h = ws["emb"][torch.tensor(ids)].float()
    for L in range(2):
        x = P.rms_norm(h, ws[f"n{L}a"], eps)
        proj = x @ ws[f"m{L}"].float().T
        s, outs = torch.zeros(h.shape[1]), []
        for t in range(len(ids)):
            s = s * decay + proj[t]
            outs.append(s / (t + 1))
        h = h + torch.stack(outs)
        x = P.rms_norm(h, ws[f"n{L}b"], eps)
        pick = (x[:, :1] > 0).float()
        h = h + x * (pick * scales[0] + (1 - pick) * scales[1])
    return P.rms_norm(h, ws["nf"], eps) @ ws["emb"].float().T


def test_toy_mixer_with_state_registers_builds_and_steps():
    from quanta_b200.engine.model import Model
    from quanta_b200.engine.step import Engine
    from quanta_b200.parts.spec import ModelSpec
    from quanta_b200.weights import DictSource, RandomSource
    _register_toys()
    Hd, V, eps, decay, scales = 40, 97, 1e-5, 0.9, (0.5, -0.25)
    norm = lambda n: ("rms_norm", dict(width=Hd, eps=eps, weight_name=n))      # noqa: E731
    layers = [("pre_norm", dict(hidden_size=Hd, mixer=("toy_running_mean", dict(hidden_size=Hd, weight_name=f"m{L}", decay=decay)),
                                feed_forward=("toy_two_way_routing", dict(hidden_size=Hd, scales=scales)),
                                mixer_norm=norm(f"n{L}a"), feed_forward_norm=norm(f"n{L}b"))) for L in range(2)]
    spec = ModelSpec(name="toy", vocab_size=V, hidden_size=Hd, embedding_name="emb", layers=layers,
                     final_norm=norm("nf"), head_name=None, tied_head=True)
    model = Model(spec, dtype="float32")
    src = RandomSource(model.tensor_specs(), seed=3, matrix_dtype=torch.float32)
    ws = {n: src.read(n, "cpu") for n in src.names()}
    model.load(DictSource(ws))
    eng = Engine(model, num_pages=4, page_size=4, max_requests=3)
    assert eng.manager.groups == [] and set(eng.state[0]) == {"sum", "count"}     # no pages, but state slots
    reqs = {"a": H.random_tokens(19, V, 1), "b": H.random_tokens(11, V, 2), "c": H.random_tokens(7, V, 3)}
    want = {}
    for rid, toks in reqs.items():
        lg = _toy_plain(ws, toks, decay, scales, eps)
        want.update({(rid, i): lg[i] for i in range(len(toks))})
    for cut in (H.cut_whole(reqs), H.cut_portions(reqs), H.cut_mixed(reqs, 3, seed=2), H.cut_mixed(reqs, 2, seed=9)):
        got = H.replay(eng, cut)       # a slot is zeroed when the next request takes it
        assert H.first_wrong(got, want, 1e-4) is None


def _register_cache_toys():
    from dataclasses import dataclass
    from quanta_b200.parts.base import CacheSpec, CacheStream, Embedding, Head, Mixer, Retention, TensorSpec, register

    @dataclass(frozen=True)
    class SinksAndWindow(Retention):
        """The first ``sinks`` positions stay readable for ever, beside a window of the last ``window``."""
        sinks: int = 4
        window: int = 8

        def needed_ranges(self, length):
            return [(0, self.sinks), (max(0, length - self.window + 1), None)]

    @register("mixer", "toy_latent_attention")
    class LatentAttention(Mixer):
        """Attention over ONE cached stream: each token leaves a 24-wide vector that serves as key and as
        value (no second stream), read by later tokens at the first ``sinks`` positions and inside a window."""

        def __init__(self, hidden_size, width, sinks, window, names):
            self.H, self.W, self.sinks, self.window, self.names = hidden_size, width, sinks, window, names
            self.down = self.q = self.up = None

        def tensor_specs(self):
            n = self.names
            return [TensorSpec(n["down"], (self.W, self.H)), TensorSpec(n["q"], (self.W, self.H)),
                    TensorSpec(n["up"], (self.H, self.W))]

        def load(self, fetch):
            self.down, self.q, self.up = (fetch(self.names[k]) for k in ("down", "q", "up"))

        def cache_spec(self):
            return CacheSpec((CacheStream("latent", 1, self.W),), SinksAndWindow(self.sinks, self.window))

        def forward(self, x, ctx, cache, state):
            pages, ps = cache.streams["latent"], cache.page_size         # [num_pages, 1, page_size, W]
            c = x.float() @ self.down.float().T
            q = x.float() @ self.q.float().T
            out = torch.empty_like(c)
            starts, after = ctx.host["req_start"], ctx.host["req_len_after"]
            table = cache.block_table.cpu()
            for r in range(len(starts) - 1):                              # a toy: plain torch, a token at a time
                t0, n = starts[r], starts[r + 1] - starts[r]
                first = after[r] - n
                for i in range(n):
                    p = first + i
                    pages[int(table[r, p // ps]), 0, p % ps] = c[t0 + i].to(pages.dtype)
                for i in range(n):
                    p = first + i
                    keys = [j for j in range(p + 1) if j < self.sinks or j > p - self.window]
                    assert all(int(table[r, j // ps]) >= 0 for j in keys), "a page the rule needs was given back"
                    cj = torch.stack([pages[int(table[r, j // ps]), 0, j % ps] for j in keys]).float()
                    w = torch.softmax((cj @ q[t0 + i]) * self.W ** -0.5, 0)
                    out[t0 + i] = w @ cj
            return (out @ self.up.float().T).to(x.dtype)

    @register("embedding", "toy_scaled_table")
    class ScaledTable(Embedding):
        def __init__(self, vocab_size, hidden_size, weight_name, scale):
            self.V, self.H, self.weight_name, self.scale = vocab_size, hidden_size, weight_name, scale

        def tensor_specs(self):
            return [TensorSpec(self.weight_name, (self.V, self.H))]

        def load(self, fetch):
            self.table = fetch(self.weight_name)

        def forward(self, ids, ctx):
            return self.table[ids.long()].float() * self.scale

    @register("head", "toy_scaled_head")
    class ScaledHead(Head):
        """Logits times a constant, from the embedding table; the pending sum and the norm in plain torch."""

        def __init__(self, vocab_size, hidden_size, table_name, norm_name, eps, logit_scale):
            self.V, self.H, self.table_name, self.norm_name = vocab_size, hidden_size, table_name, norm_name
            self.eps, self.logit_scale = eps, logit_scale

        def tensor_specs(self):
            return [TensorSpec(self.table_name, (self.V, self.H)), TensorSpec(self.norm_name, (self.H,), "f32", "gain")]

        def load(self, fetch):
            self.table, self.gain = fetch(self.table_name), fetch(self.norm_name)

        def forward(self, h, pending, rows, ctx):
            x = h[rows.long()]
            if pending is not None:
                add = pending[rows.long()].float()
                x = x + (add if add.dim() == 2 else add.sum(1))
            x = self.gain * x * torch.rsqrt((x * x).mean(-1, keepdim=True) + self.eps)
            return (x @ self.table.float().T) * self.logit_scale


def _cache_toy_plain(ws, ids, cfg):
    """Whole-sequence plain version: scaled embedding, [norm, latent attention, norm, two-way] x 2, scaled head."""
    T = len(ids)
    h = ws["emb"][torch.tensor(ids)].float() * cfg["emb_scale"]
    j, p = torch.arange(T)[None, :], torch.arange(T)[:, None]
    mask = (j <= p) & ((j < cfg["sinks"]) | (j > p - cfg["window"]))
    for L in range(2):
        x = P.rms_norm(h, ws[f"n{L}a"], cfg["eps"])
        c, q = x @ ws[f"down{L}"].float().T, x @ ws[f"q{L}"].float().T
        s = ((q @ c.T) * cfg["width"] ** -0.5).masked_fill(~mask, float("-inf"))
        h = h + (torch.softmax(s, -1) @ c) @ ws[f"up{L}"].float().T
        x = P.rms_norm(h, ws[f"n{L}b"], cfg["eps"])
        pick = (x[:, :1] > 0).float()
        h = h + x * (pick * cfg["scales"][0] + (1 - pick) * cfg["scales"][1])
    return (P.rms_norm(h, ws["nf"], cfg["eps"]) @ ws["emb"].float().T) * cfg["logit_scale"]


def test_toy_cache_stream_retention_rule_embedding_and_head():
    """What a new architecture may bring without a change to the framework's files: a mixer that keeps one
    stream of its own width instead of keys and values, a rule of its own for which positions stay readable
    (the first four and a window; the manager gives the pages between back), an embedding and an output
    head of its own.  Built from a specification, stepped under the four cuttings with as few pages as the
    rule allows, against the whole-sequence plain version."""
    from quanta_b200.engine.model import Model
    from quanta_b200.engine.step import Engine
    from quanta_b200.parts.spec import ModelSpec
    from quanta_b200.weights import DictSource, RandomSource
    _register_toys()
    _register_cache_toys()
    cfg = dict(eps=1e-5, sinks=4, window=9, width=24, scales=(0.5, -0.25), emb_scale=3.0, logit_scale=0.25)
    Hd, V = 40, 97
    norm = lambda n: ("rms_norm", dict(width=Hd, eps=cfg["eps"], weight_name=n))      # noqa: E731
    layers = [("pre_norm", dict(hidden_size=Hd, mixer=("toy_latent_attention", dict(
        hidden_size=Hd, width=cfg["width"], sinks=cfg["sinks"], window=cfg["window"],
        names={"down": f"down{L}", "q": f"q{L}", "up": f"up{L}"})),
        feed_forward=("toy_two_way_routing", dict(hidden_size=Hd, scales=cfg["scales"])),
        mixer_norm=norm(f"n{L}a"), feed_forward_norm=norm(f"n{L}b"))) for L in range(2)]
    spec = ModelSpec(name="cache toy", vocab_size=V, hidden_size=Hd, embedding_name="emb", layers=layers,
                     final_norm=norm("nf"), head_name=None, tied_head=True,
                     embedding=("toy_scaled_table", dict(vocab_size=V, hidden_size=Hd, weight_name="emb", scale=cfg["emb_scale"])),
                     head=("toy_scaled_head", dict(vocab_size=V, hidden_size=Hd, table_name="emb", norm_name="nf",
                                                   eps=cfg["eps"], logit_scale=cfg["logit_scale"])))
    model = Model(spec, dtype="float32")
    assert [s.name for s in model.tensor_specs()].count("emb") == 1            # asked for twice, loaded once
    src = RandomSource(model.tensor_specs(), seed=4, matrix_dtype=torch.float32)
    ws = {n: src.read(n, "cpu") for n in src.names()}
    model.load(DictSource(ws))
    assert model.head.table is model.embedding.table
    reqs = {"a": H.random_tokens(61, V, 1), "b": H.random_tokens(33, V, 2), "c": H.random_tokens(47, V, 3)}
    want = {}
    for rid, toks in reqs.items():
        lg = _cache_toy_plain(ws, toks, cfg)
        want.update({(rid, i): lg[i] for i in range(len(toks))})
    page = 4
    for what, cut in (("whole", H.cut_whole(reqs)), ("tail", H.cut_tail_decode(reqs, 32)),
                      ("portions", H.cut_portions(reqs)), ("mixed", H.cut_mixed(reqs, 3, seed=2))):
        eng = Engine(model, num_pages=H.tokens_in_flight(cut, page) // page, page_size=page, max_requests=3)
        assert not eng.use_graphs                                 # the toy reads host copies
        (group,) = eng.manager.groups
        assert [(s.name, s.heads, s.width) for s in group.spec.streams] == [("latent", 1, 24)]
        assert set(eng.kv[0]) == {"latent"} and eng.kv[0]["latent"].shape[1:] == (1, page, 24)
        got = H.replay(eng, cut)
        eng.manager.check_invariants()
        assert H.first_wrong(got, want, 1e-4) is None, (what, H.worst_error(got, want))
        if what != "whole":
            # decoding request a to 61 tokens never held more than the sinks' page, the window's and the step's
            assert group.pool.high_water < sum(-(-len(t) // page) for t in reqs.values())


def test_toy_position_encoding_in_the_real_attention(model_dirs):
    """The attention mixer takes any registered position encoding: here a linear frequency ladder."""
    from quanta_b200.parts.attention import GQAttention
    from quanta_b200.parts.base import LayerCache
    _register_toys()
    torch.manual_seed(5)
    Hd, nq, nkv, hd, rd, T = 48, 4, 2, 16, 8, 11
    ws = {n: 0.2 * torch.randn(*s) for n, s in [("q", (nq * hd, Hd)), ("k", (nkv * hd, Hd)), ("v", (nkv * hd, Hd)), ("o", (Hd, nq * hd))]}
    att = GQAttention(Hd, nq, nkv, hd, hd ** -0.5, ("toy_linear_ladder", dict(rotary_dim=rd)), None, 1e-6,
                      {"q": "q", "k": "k", "v": "v", "o": "o"})
    att.load(lambda n: ws[n].to(DEV))
    x = torch.randn(T, Hd)
    kc = torch.zeros(3, nkv, 4, hd, device=DEV)
    cache = LayerCache(kc, torch.zeros_like(kc), 4, torch.arange(3, dtype=torch.int32, device=DEV).view(1, -1))
    got = att.forward(x.to(DEV), _ctx(T), cache, {})
    inv = 1.0 - torch.arange(rd // 2, dtype=torch.float32) / (rd // 2)

    def rope(t):
        ang = torch.arange(T, dtype=torch.float32)[:, None] * inv[None]
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        a, b = t[..., : rd // 2], t[..., rd // 2: rd]
        return torch.cat([a * c - b * s, b * c + a * s, t[..., rd:]], -1)
    q = rope((x @ ws["q"].T).reshape(T, nq, hd))
    k = rope((x @ ws["k"].T).reshape(T, nkv, hd))
    v = (x @ ws["v"].T).reshape(T, nkv, hd)
    want = P.causal_attention(q, k, v, None, torch.float32) @ ws["o"].T
    assert torch.allclose(got.cpu(), want, atol=2e-5)


# ---- generation through the entry point ------------------------------------------------------------------
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("C", "bfloat16"), ("D", "float32"),
                                        ("D", "bfloat16")])
def test_greedy_generation_matches_plain(model_dirs, plain_models, name, dtype):
    from quanta_b200 import generate
    from quanta_b200.engine.generate import LLM
    weights, cfg = plain_models[name]
    vocab = TINY[name]["vocab_size"]
    prompts = [H.random_tokens(n, vocab, 40 + i) for i, n in enumerate((5, 11, 16))]
    llm = LLM(model_dirs[name], dtype=dtype, page_size=4, num_pages=40, max_requests=4, max_step_tokens=12, prefill_chunk=6)
    got = generate(llm, prompts, max_new_tokens=8, eos_id=[])
    act = None if dtype == "float32" else torch.bfloat16
    for p, g in zip(prompts, got):
        want = P.generate(weights, cfg, p, max_new_tokens=8, act=act)
        if dtype == "float32":
            assert g == want
        else:
            # bfloat16: the first token must agree unless the top two logits are within rounding
            lg = P.forward_logits(weights, cfg, p, act=act)[-1]
            top2 = torch.topk(lg, 2).values
            assert g[0] == want[0] or float(top2[0] - top2[1]) < 0.02
    one = generate(llm, prompts[1], max_new_tokens=8, eos_id=[])
    assert one == got[1]                                       # alone or in a batch: the same tokens
    with pytest.raises(ValueError, match="empty"):
        generate(llm, [], max_new_tokens=2)
    assert llm.engine.manager.stats()["live_requests"] == 0


def test_sampled_generation_is_seeded_and_matches_plain(model_dirs, plain_models):
    from quanta_b200 import generate
    from quanta_b200.engine.generate import LLM
    name = "B"
    weights, cfg = plain_models[name]
    prompts = [H.random_tokens(7, 1000, 1), H.random_tokens(23, 1000, 2)]
    llm = LLM(model_dirs[name], dtype="float32", page_size=8, num_pages=16, max_requests=2, max_step_tokens=8, prefill_chunk=6)
    kw = dict(max_new_tokens=6, temperature=0.8, seed=1234, eos_id=[])
    a = generate(llm, prompts, **kw)
    b = generate(llm, prompts, **kw)
    c = generate(llm, prompts, **{**kw, "seed": 99})
    assert a == b and a != c
    for p, g in zip(prompts, a):
        assert g == P.generate(weights, cfg, p, max_new_tokens=6, temperature=0.8, seed=1234)
    d = generate(llm, prompts[0], max_new_tokens=6, temperature=0.8, seed=1234, top_k=20, top_p=0.9, min_p=0.01,
                 repetition_penalty=1.3, presence_penalty=0.2, frequency_penalty=0.1, eos_id=[])
    assert d == P.generate(weights, cfg, prompts[0], max_new_tokens=6, temperature=0.8, seed=1234, top_k=20, top_p=0.9,
                           min_p=0.01, repetition_penalty=1.3, presence_penalty=0.2, frequency_penalty=0.1)


def test_eos_and_few_pages(model_dirs, plain_models):
    """An eos id ends a request and is not returned; with too few pages requests are preempted and
    recomputed, and the tokens are the same as with plenty."""
    from quanta_b200 import generate
    from quanta_b200.engine.generate import LLM
    name = "A"
    weights, cfg = plain_models[name]
    prompts = [H.random_tokens(9, 512, 70 + i) for i in range(3)]
    roomy = LLM(model_dirs[name], dtype="float32", page_size=4, num_pages=64, max_requests=4)
    want = generate(roomy, prompts, max_new_tokens=12, eos_id=[])
    tight = LLM(model_dirs[name], dtype="float32", page_size=4, num_pages=11, max_requests=4, prefill_chunk=8)
    got = generate(tight, prompts, max_new_tokens=12, eos_id=[])
    assert got == want and tight.last_stats["preemptions"] >= 1
    stop = want[0][4]
    cut = generate(roomy, prompts[0], max_new_tokens=12, eos_id=stop)
    assert cut == want[0][: want[0].index(stop)]
    # sampled: a request that is preempted and recomputed goes on with the draw number it had reached,
    # so the tokens are those of the plain implementation whether or not anything was preempted
    kw = dict(max_new_tokens=12, temperature=0.8, seed=4321, top_k=40, eos_id=[])
    drawn = generate(tight, prompts, **kw)
    assert tight.last_stats["preemptions"] >= 1
    assert drawn == generate(roomy, prompts, **kw)
    for p, g in zip(prompts, drawn):
        assert g == P.generate(weights, cfg, p, max_new_tokens=12, temperature=0.8, seed=4321, top_k=40)


def test_state_slots_on_the_device(model_dirs):
    """Every live request has a record on the device: position, prompt length, draws so far, the last
    sampled token, seed and options.  After steps that mix prompt portions, single tokens, sampling with
    three different option sets and a request that ends, the records say what the host's bookkeeping says,
    the freed slot is zero, and a record that disagrees with the host is reported."""
    import struct
    from quanta_b200 import kernels
    from quanta_b200.engine.model import load_model
    from quanta_b200.engine.scheduler import SamplingParams
    from quanta_b200.engine.step import Engine, StepEntry
    from quanta_b200.sampling.sampler import Sampler

    class Req:
        def __init__(self, rid, prompt, params):
            self.rid, self.prompt, self.params, self.generated = rid, prompt, params, []

    model, _ = load_model(model_dirs["A"], dtype="float32")
    eng = Engine(model, num_pages=64, page_size=4, max_requests=4)
    sampler = Sampler(DEV)
    reqs = {"a": Req("a", H.random_tokens(9, 512, 1), SamplingParams(temperature=0.8, seed=5, top_k=20)),
            "b": Req("b", H.random_tokens(14, 512, 2), SamplingParams(temperature=0.0)),
            "c": Req("c", H.random_tokens(6, 512, 3), SamplingParams(temperature=1.1, seed=2 ** 35 + 1, top_p=0.9, min_p=0.01))}

    def step(parts, end=()):
        """parts: (request, tokens, samples?)"""
        for r, _, _ in parts:
            if not eng.manager.has(r.rid):
                eng.admit(r.rid, prompt_len=len(r.prompt), params=r.params, drawn=len(r.generated))
        entries = [StepEntry(r.rid, toks, (len(toks) - 1,) if samples else ()) for r, toks, samples in parts]
        logits = eng.step(entries, end=end)
        who = [r for r, _, samples in parts if samples]
        if who:
            for r, t in zip(who, sampler.sample(logits, eng.slots, eng.last_want_slots, who, eng.status)):
                r.generated.append(t)

    a, b, c = reqs["a"], reqs["b"], reqs["c"]
    step([(a, a.prompt, True), (b, b.prompt[:5], False)])
    step([(a, a.generated[-1:], True), (b, b.prompt[5:], True), (c, c.prompt, True)])
    for _ in range(5):
        step([(r, r.generated[-1:], True) for r in (a, b, c)])      # from captured graphs after the first
    slot_of = {r.rid: eng.manager.slot(r.rid) for r in (a, b, c)}
    step([(a, a.generated[-1:], True), (c, c.generated[-1:], True)], end=["b"])
    rec = eng.slots.cpu()
    bits = lambda x: struct.unpack("<i", struct.pack("<f", x))[0]      # noqa: E731
    for r in (a, c):
        row = rec[slot_of[r.rid]].tolist()
        assert row[kernels.SLOT_LIVE] == 1
        assert row[kernels.SLOT_POSITION] == eng.manager.length(r.rid) == len(r.prompt) + len(r.generated) - 1
        assert row[kernels.SLOT_PROMPT] == len(r.prompt) and row[kernels.SLOT_DRAWN] == len(r.generated)
        assert row[kernels.SLOT_LAST] == r.generated[-1]
        assert (row[kernels.SLOT_SEED_LO], row[kernels.SLOT_SEED_HI]) == (r.params.seed & 0xFFFFFFFF, r.params.seed >> 32)
        assert row[kernels.SLOT_TOP_K] == r.params.top_k and row[kernels.SLOT_TEMPERATURE] == bits(r.params.temperature)
        assert row[kernels.SLOT_TOP_P] == bits(r.params.top_p) and row[kernels.SLOT_MIN_P] == bits(r.params.min_p)
    assert len(a.generated) == 8 and len(c.generated) == 7
    assert rec[slot_of["b"]].tolist() == [0] * kernels.SLOT_WORDS
    free = [s for s in range(4) if s not in (slot_of["a"], slot_of["c"])]
    assert rec[free].abs().sum() == 0
    # the device's record and the host's bookkeeping are compared at every step
    eng.slots[slot_of["a"], kernels.SLOT_POSITION] += 1
    eng.step([StepEntry("a", a.generated[-1:], ())])
    with pytest.raises(kernels.KernelError, match="state slot"):
        eng.check()


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("C", "bfloat16")])
def test_steps_launched_ahead_give_the_same_tokens(model_dirs, name, dtype):
    """Decode steps are launched before the host has read the tokens of the step before (their ids stay on
    the device).  With that switched off the same tokens must come out: greedy and sampled, with requests
    of different lengths, with a request that stops on an end token in the middle (its token of the step
    ahead is dropped) and with penalties (which need the tokens on the host: no step ahead then)."""
    from quanta_b200.engine.generate import LLM
    from quanta_b200.engine.scheduler import SamplingParams
    vocab = TINY[name]["vocab_size"]
    prompts = [H.random_tokens(5 + 3 * i, vocab, 300 + i) for i in range(4)]
    llm = LLM(model_dirs[name], dtype=dtype, page_size=4, num_pages=96, max_requests=4, prefill_chunk=8)

    def both(params):
        llm.lookahead = True
        ahead = llm.generate(prompts, params)
        n_ahead = llm.last_stats["steps_ahead"]
        log = list(llm.step_log)
        llm.lookahead = False
        plain_order = llm.generate(prompts, params)
        assert ahead == plain_order and llm.last_stats["steps_ahead"] == 0
        return ahead, log, n_ahead

    lengths = [SamplingParams(max_new_tokens=n, temperature=0.0) for n in (40, 7, 23, 31)]
    greedy, log, n_ahead = both(lengths)
    assert [len(g) for g in greedy] == [40, 7, 23, 31] and n_ahead >= 20
    assert sum(e["sampled"] for e in log) >= 40 + 7 + 23 + 31          # steps ahead may sample a token that is dropped
    stop = greedy[0][17]
    cut, _, _ = both([SamplingParams(max_new_tokens=40, temperature=0.0, eos_token_ids=(stop,))] + lengths[1:])
    assert cut[0] == greedy[0][: greedy[0].index(stop)] and cut[1:] == greedy[1:]
    sampled, _, _ = both([SamplingParams(max_new_tokens=20, temperature=0.9, top_k=50, seed=7 + i) for i in range(4)])
    assert len({tuple(x) for x in sampled}) == 4
    _, _, n_ahead = both([SamplingParams(max_new_tokens=12, temperature=0.7, seed=3, repetition_penalty=1.2,
                                         presence_penalty=0.1)] * 4)
    assert n_ahead == 0


def test_more_q_heads_per_kv_head_than_the_decode_kernel_takes(tmp_path):
    """72 q heads on one kv head: single tokens run as portions of one (no captured decode step); and a
    head size of 80 beside it (no TMA boxes, no tcgen05 attention).  Both against the plain implementation,
    decoding token by token after a prompt."""
    from safetensors.torch import load_file
    from quanta_b200.config import MiniMaxM3Config
    from quanta_b200.engine.model import load_model, write_random_model
    from quanta_b200.engine.step import Engine
    common = dict(architectures=["MiniMaxM3ForCausalLM"], model_type="minimax_m3", rms_norm_eps=1e-6,
                  tie_word_embeddings=False, num_hidden_layers=1, use_routing_bias=True, use_qk_norm=True)
    cases = {
        "wide_group": dict(vocab_size=400, hidden_size=256, intermediate_size=128, num_attention_heads=72,
                           num_key_value_heads=1, head_dim=128, rotary_dim=64, rope_theta=5e6, qk_norm_type="per_layer",
                           num_local_experts=8, num_experts_per_tok=2),
        "head_80": dict(vocab_size=1001, hidden_size=120, intermediate_size=72, num_attention_heads=5,
                        num_key_value_heads=5, head_dim=80, rotary_dim=40, rope_theta=1e4, qk_norm_type="per_head",
                        num_local_experts=5, num_experts_per_tok=5),
    }
    for name, raw in cases.items():
        raw = dict(common, **raw)
        d = tmp_path / name
        write_random_model(MiniMaxM3Config.from_dict(raw), 5, d)
        plain = (load_file(str(d / "model.safetensors")), P.read_config(d))
        reqs = {"a": H.random_tokens(150, raw["vocab_size"], 1), "b": H.random_tokens(70, raw["vocab_size"], 2)}
        want = H.plain_logits(plain, reqs, act=torch.bfloat16)
        exact = H.plain_logits(plain, reqs)
        tol = 2.0 * max(float((want[k] - exact[k]).abs().max()) for k in want)
        model, _ = load_model(d, dtype="bfloat16")
        eng = Engine(model, num_pages=32, page_size=16, max_requests=4)
        assert eng.use_graphs == (name != "wide_group")
        for cut in (H.cut_tail_decode(reqs, 40), H.cut_mixed(reqs, 2, seed=4)):
            got = H.replay(eng, cut)
            assert H.first_wrong(got, want, tol) is None, (name, H.worst_error(got, want), tol)


def test_command_line(model_dirs):
    cmd = [sys.executable, "-m", "quanta_b200", "generate", "--model", str(model_dirs["A"]), "--dtype", "float32",
           "--prompt-ids", "5,17,3", "--max-new-tokens", "4", "--block-size", "4", "--num-pages", "16", "--eos-id", "600"]
    r = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    toks = [int(t) for t in r.stdout.strip().split(",")]
    from quanta_b200 import generate
    assert toks == generate(str(model_dirs["A"]), [5, 17, 3], max_new_tokens=4, dtype="float32", page_size=4, num_pages=16, eos_id=[])
