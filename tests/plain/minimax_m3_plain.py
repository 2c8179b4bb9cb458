"""Plain, slow implementation of the MiniMax-M3 text decoder (MiniMax-M2-family layer math).

Whole sequences, no cache, one function for each part, plain PyTorch (on the CPU; on a CUDA device
when the tensors it is given live there, for the layer widths of the full-size model).  It shares no
code with the ``quanta_b200`` package: it reads the raw ``config.json`` dictionary and the tensors by
checkpoint name (a dictionary, or a function ``name -> tensor`` so that one layer's tensors can be made
or read when the layer runs and dropped after it), and is the oracle the engine's tests compare against.

This file rests on the reference's formulas (pmrjge/quanta); each function cites the file and
lines it restates.  The reference's own model code needs ``mlx`` and cannot be imported on this
machine; its pure-numpy oracle functions and its config parser can, and ``tests/golden`` holds
the comparison of this file with those.

``act`` is the dtype activations are rounded to where the reference keeps them in the compute
dtype (``None``: no rounding, everything stays in ``compute``).  Softmax, norm statistics, router
logits, rotation angles and the residual sum stay in ``compute`` (float32 or float64).
"""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

# ----------------------------------------------------------------------------------------------
# configuration (own reading of config.json; src/quanta/minimax/config.py:136-188,
# src/quanta/minimax/config_m3.py:223-255 for text_config / partial_rotary_factor)
# ----------------------------------------------------------------------------------------------


def read_config(model_dir) -> dict:
    raw = json.loads((Path(model_dir) / "config.json").read_text())
    return normalise_config(raw)


def normalise_config(raw: dict) -> dict:
    c = dict(raw.get("text_config", raw))
    hd = int(c["head_dim"])
    rd = c.get("rotary_dim")
    if rd is None:
        rd = int(round(hd * float(c.get("partial_rotary_factor", 1.0))))
    out = {
        "V": int(c["vocab_size"]), "H": int(c["hidden_size"]), "I": int(c["intermediate_size"]),
        "L": int(c["num_hidden_layers"]), "nq": int(c["num_attention_heads"]),
        "nkv": int(c["num_key_value_heads"]), "hd": hd, "rd": int(rd),
        "theta": float(c.get("rope_theta", 1e6)),
        "qk_norm": bool(c.get("use_qk_norm", False)),
        "qk_norm_type": str(c.get("qk_norm_type", "per_layer")),
        "E": int(c["num_local_experts"]), "k": int(c["num_experts_per_tok"]),
        "bias": bool(c.get("use_routing_bias", True)),
        "renorm": bool(c.get("norm_topk_prob", True)),
        "scale": float(c.get("routed_scaling_factor", 1.0)),
        "eps": float(c.get("rms_norm_eps", 1e-6)),
        "tied": bool(c.get("tie_word_embeddings", False)),
    }
    return out


# ----------------------------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------------------------


def _round(x: torch.Tensor, act, compute) -> torch.Tensor:
    return x if act is None else x.to(act).to(compute)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """``w * x * rsqrt(mean(x^2) + eps)`` over the last axis (src/quanta/minimax/model_m3.py:60-65)."""
    return w.to(x.dtype) * (x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps))


def embedding(ids: torch.Tensor, table: torch.Tensor, compute) -> torch.Tensor:
    """``h = embed[ids]`` (src/quanta/minimax/model.py:91)."""
    return table[ids.long()].to(compute)


def linear(x: torch.Tensor, w: torch.Tensor, act, compute) -> torch.Tensor:
    """``x @ w.T`` without bias (src/quanta/minimax/attention.py:166-169); result rounded to ``act``."""
    return _round(x @ w.to(compute).T, act, compute)


def qk_norm(q: torch.Tensor, w: torch.Tensor, n_heads: int, hd: int, kind: str, eps: float) -> torch.Tensor:
    """q/k RMSNorm before the rotation.  ``per_layer``: one statistic over the concatenated heads,
    weight ``[n_heads*hd]`` (src/quanta/minimax/model_m3.py:15-17 names this the M2 form);
    ``per_head``: statistic over each head's ``hd`` dims, weight ``[hd]`` shared by the heads
    (src/quanta/minimax/attention.py:172-182)."""
    T = q.shape[0]
    if kind == "per_layer":
        return rms_norm(q.reshape(T, n_heads * hd), w, eps).reshape(T, n_heads, hd)
    if kind == "per_head":
        return rms_norm(q.reshape(T, n_heads, hd), w, eps)
    raise ValueError(kind)


def rope_inv_freq(rd: int, theta: float) -> torch.Tensor:
    """``1 / theta**(2i/rd)`` in float32 (src/quanta/minimax/model_m3.py:68-72)."""
    return 1.0 / (theta ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))


def partial_rope(x: torch.Tensor, pos: torch.Tensor, rd: int, theta: float) -> torch.Tensor:
    """Rotate-half on the first ``rd`` dims of each head, the rest unchanged
    (src/quanta/minimax/model_m3.py:83-96, src/quanta/minimax/attention.py:120-135).
    ``x`` ``[T, heads, hd]``; ``pos`` ``[T]`` absolute positions.  The angle is the float32
    product ``pos * inv_freq``."""
    inv = rope_inv_freq(rd, theta).to(x.device)
    ang = (pos.to(device=x.device, dtype=torch.float32)[:, None] * inv[None, :]).to(x.dtype)        # [T, rd/2]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x1, x2 = x[..., : rd // 2], x[..., rd // 2: rd]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin, x[..., rd:]], dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, act, compute, window=None) -> torch.Tensor:
    """Causal softmax attention of one whole sequence with grouped heads
    (src/quanta/minimax/attention.py:194-203, mask :105-110).  ``q`` ``[T,nq,hd]``, ``k``/``v``
    ``[T,nkv,hd]``; q head ``h`` reads kv head ``h // (nq/nkv)``; scale ``hd**-0.5``; the softmax is
    taken in ``compute`` and the probabilities are rounded to ``act`` before ``P @ V``.
    ``window`` (not in the reference, whose layers all read every key; used by the tests of cache groups):
    a query at position p reads the keys p-window+1 .. p only."""
    T, nq, hd = q.shape
    rep = nq // k.shape[1]
    kr = k.repeat_interleave(rep, dim=1).transpose(0, 1)          # [nq,T,hd]
    vr = v.repeat_interleave(rep, dim=1).transpose(0, 1)
    s = (q.transpose(0, 1) @ kr.transpose(1, 2)) * (hd ** -0.5)   # [nq,T,T]
    mask = torch.ones(T, T, dtype=torch.bool, device=q.device).tril()
    if window:
        mask &= ~torch.ones(T, T, dtype=torch.bool, device=q.device).tril(-int(window))
    s = s.masked_fill(~mask, float("-inf"))
    p = _round(torch.softmax(s, dim=-1), act, compute)
    out = (p @ vr).transpose(0, 1).reshape(T, nq * hd)
    return _round(out, act, compute)


def router(x: torch.Tensor, gate_w: torch.Tensor, bias, k: int, renorm: bool, scale: float, given=None):
    """Sigmoid scores, bias for selection only, top-k, bias-free weights renormalised and scaled
    (src/quanta/minimax/moe.py:36-56).  Ties are broken towards the lower expert index.
    Returns ``(idx [T,k] int64 sorted by choice descending, w [T,k])``.  ``given`` ``[T,k]``: the choice
    is taken from there instead (to follow another implementation through a near tie); the weights
    are still this function's scores of those experts."""
    logits = x @ gate_w.to(x.dtype).T
    scores = torch.sigmoid(logits)
    choice = scores + bias.to(x.dtype)[None] if bias is not None else scores
    idx = torch.argsort(-choice, dim=-1, stable=True)[:, :k] if given is None else given.to(x.device).long()
    w = torch.gather(scores, 1, idx)
    if k > 1 and renorm:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return idx, w * scale


def router_margin(x: torch.Tensor, gate_w: torch.Tensor, bias, k: int) -> torch.Tensor:
    """How far each token is from choosing other experts: the k-th largest choice score minus the
    (k+1)-th (src/quanta/minimax/moe.py:44-52 for the scores).  A token whose margin is within the
    rounding of the scores may choose differently in another implementation of the same arithmetic."""
    scores = torch.sigmoid(x @ gate_w.to(x.dtype).T)
    choice = scores + bias.to(x.dtype)[None] if bias is not None else scores
    if k >= choice.shape[-1]:
        return torch.full((x.shape[0],), float("inf"), dtype=x.dtype, device=x.device)
    top = torch.topk(choice, k + 1, dim=-1).values
    return top[:, k - 1] - top[:, k]


def expert_swiglu(x: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor, w2: torch.Tensor, act, compute):
    """``down(silu(gate(x)) * up(x))`` with ``w1`` gate, ``w3`` up, ``w2`` down
    (src/quanta/minimax/moe.py:59-70)."""
    g = x @ w1.to(compute).T
    u = x @ w3.to(compute).T
    a = _round(g * torch.sigmoid(g) * u, act, compute)
    return a @ w2.to(compute).T


def moe(x: torch.Tensor, gate_w, bias, experts, k, renorm, scale, act, compute, given=None, probe=None) -> torch.Tensor:
    """Routed sum of the chosen experts, weights applied after ``down``, accumulated in ``compute``;
    no shared expert (src/quanta/minimax/moe.py:73-88).  ``experts(e)`` or ``experts[e]`` ``= (w1, w3, w2)``.  The loop goes
    over the experts, each taking the tokens that chose it (as moe.py:84-88 does with ``idx_flat``).
    ``given``: see ``router``.  ``probe``: a dictionary that receives the choice (``idx``)."""
    idx, w = router(x, gate_w, bias, k, renorm, scale, given)
    if probe is not None:
        probe["idx"] = idx
    out = torch.zeros_like(x)
    for e in sorted(set(idx.reshape(-1).tolist())):
        tok, slot = torch.nonzero(idx == e, as_tuple=True)
        y = expert_swiglu(x[tok], *(experts(e) if callable(experts) else experts[e]), act, compute)
        out.index_add_(0, tok, w[tok, slot][:, None] * y)
    return out


# ----------------------------------------------------------------------------------------------
# the block and the model
# ----------------------------------------------------------------------------------------------


def _w(weights, name: str) -> torch.Tensor:
    """``weights``: tensors by checkpoint name, or a function that returns the tensor of a name."""
    if callable(weights):
        return weights(name)
    if name in weights:
        return weights[name]
    return weights["language_model." + name]


def block(h, pos, weights, cfg, layer: int, act, compute, weight_layer: int | None = None, window=None,
          probe: dict | None = None, given=None, kv_of: dict | None = None):
    """``h + attn(norm(h))`` then ``h + moe(norm(h))`` (src/quanta/minimax/model.py:70-73).
    ``probe``: a dictionary that receives this layer's ``router_margin`` of every token, the experts
    chosen and the keys and values it cached (``margin``, ``idx``, ``k``, ``v``).  ``given``: the experts to
    take instead of the router's own choice.  ``kv_of``: another run of a block (its ``probe``): this one
    attends over THAT run's cached keys and values with its own queries and caches none (not in the
    reference, whose layers each keep their own; used by the tests of the run order)."""
    c = cfg
    wl = layer if weight_layer is None else weight_layer
    p = f"model.layers.{wl}."
    W = lambda n: _w(weights, p + n).to(compute)      # noqa: E731
    x1 = _round(rms_norm(h, W("input_layernorm.weight"), c["eps"]), act, compute)
    T = h.shape[0]
    q = linear(x1, W("self_attn.q_proj.weight"), act, compute).reshape(T, c["nq"], c["hd"])
    k = linear(x1, W("self_attn.k_proj.weight"), act, compute).reshape(T, c["nkv"], c["hd"])
    v = linear(x1, W("self_attn.v_proj.weight"), act, compute).reshape(T, c["nkv"], c["hd"])
    if c["qk_norm"]:
        q = qk_norm(q, W("self_attn.q_norm.weight"), c["nq"], c["hd"], c["qk_norm_type"], c["eps"])
        k = qk_norm(k, W("self_attn.k_norm.weight"), c["nkv"], c["hd"], c["qk_norm_type"], c["eps"])
    q = _round(partial_rope(q, pos, c["rd"], c["theta"]), act, compute)
    k = _round(partial_rope(k, pos, c["rd"], c["theta"]), act, compute)
    if kv_of is not None:
        k, v = kv_of["k"], kv_of["v"]
    if probe is not None:
        probe["k"], probe["v"] = k, v
    a = causal_attention(q, k, v, act, compute, window)
    h = h + linear(a, W("self_attn.o_proj.weight"), act, compute)
    x2 = _round(rms_norm(h, W("post_attention_layernorm.weight"), c["eps"]), act, compute)
    m = p + "block_sparse_moe."
    experts = lambda e: tuple(_w(weights, f"{m}experts.{e}.{n}.weight") for n in ("w1", "w3", "w2"))  # noqa: E731
    bias = _w(weights, m + "e_score_correction_bias").to(compute) if c["bias"] else None
    gate_w = _w(weights, m + "gate.weight").to(compute)
    if probe is not None:
        probe["margin"] = router_margin(x2, gate_w, bias, c["k"])
    y = moe(x2, gate_w, bias, experts, c["k"], c["renorm"], c["scale"], act, compute, given=given, probe=probe)
    return h + y


def forward_logits(weights, cfg: dict, ids, *, act=None, compute=torch.float32,
                   schedule=None, windows=None, reads_cache_of=None) -> torch.Tensor:
    """Logits ``[T, V]`` of one whole sequence: embed -> blocks -> final norm -> head
    (src/quanta/minimax/model.py:86-96; head in float32, src/quanta/minimax/runtime.py:95-98).
    ``schedule`` lists the layers in the order they run (a layer may appear twice); ``windows`` maps a
    place in that order to the window of its attention (absent: every key); ``reads_cache_of`` maps a
    place to an earlier place whose cached keys and values it attends over instead of its own."""
    return forward_logits_many(weights, cfg, [ids], act=act, compute=compute, schedule=schedule, windows=windows,
                               reads_cache_of=reads_cache_of)[0]


def forward_logits_many(weights, cfg: dict, sequences, *, rows=None, act=None, compute=torch.float32,
                        schedule=None, windows=None, probes: list | None = None, given: dict | None = None,
                        reads_cache_of: dict | None = None) -> list:
    """The same for several sequences, each whole and alone, layer by layer: a layer's tensors are
    asked for once and serve every sequence, so ``weights`` may be a function that makes them when
    asked (``_LayerTensors`` keeps what one layer asked for until the next begins).  ``rows[i]``:
    the places of sequence ``i`` whose logits are returned (default: all).  The computation runs on
    the device of the embedding table.  ``probes``: a list that receives, for each sequence, one
    dictionary a layer with the tokens' ``router_margin`` and chosen experts.  ``given[(j, i)]``: the
    experts sequence ``j`` takes at place ``i`` of the layer order instead of its router's choice."""
    table = _w(weights, "model.embed_tokens.weight")
    dev = table.device
    seqs = [torch.as_tensor(s, dtype=torch.long, device=dev) for s in sequences]
    hs = [embedding(s, table, compute) for s in seqs]
    del table
    order = list(range(cfg["L"])) if schedule is None else list(schedule)
    seen = [[] for _ in hs]
    for i, wl in enumerate(order):
        layer = _LayerTensors(weights)
        for j, h in enumerate(hs):
            pos = torch.arange(h.shape[0], device=dev)
            src = (reads_cache_of or {}).get(i)
            probe = {} if (probes is not None or reads_cache_of) else None
            hs[j] = block(h, pos, layer, cfg, i, act, compute, weight_layer=wl, window=(windows or {}).get(i),
                          probe=probe, given=(given or {}).get((j, i)), kv_of=None if src is None else seen[j][src])
            seen[j].append(probe)
        del layer
    if probes is not None:
        probes.extend([{k: v for k, v in p.items() if k not in ("k", "v")} for p in per_seq] for per_seq in seen)
    norm_w = _w(weights, "model.norm.weight").to(compute)
    head = _w(weights, "model.embed_tokens.weight" if cfg["tied"] else "lm_head.weight")
    out = []
    for j, h in enumerate(hs):
        if rows is not None:
            h = h[torch.as_tensor(rows[j], dtype=torch.long, device=dev)]
        hf = _round(rms_norm(h, norm_w, cfg["eps"]), act, compute)
        out.append(hf @ head.to(compute).T)
    return out


class _LayerTensors:
    """The tensors one layer has asked ``weights`` for, kept while the layer runs on several sequences."""

    def __init__(self, weights):
        self.weights, self.kept = weights, {}

    def __call__(self, name: str) -> torch.Tensor:
        if name not in self.kept:
            self.kept[name] = _w(self.weights, name)
        return self.kept[name]


# ----------------------------------------------------------------------------------------------
# sampling (src/quanta/minimax/generate.py:34-80; penalties src/quanta/shim/omlx.py:344-363)
# ----------------------------------------------------------------------------------------------

_PHILOX_M0, _PHILOX_M1 = 0xD2511F53, 0xCD9E8D57
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85


def philox4x32(counter, key):
    """Philox-4x32-10 (Salmon et al. 2011), numpy uint64 arithmetic on 32-bit words.
    ``counter`` ``[n,4]`` uint32, ``key`` two uint32 words; returns ``[n,4]`` uint32."""
    c = np.asarray(counter, dtype=np.uint64).copy()
    k0, k1 = np.uint64(key[0]), np.uint64(key[1])
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(_PHILOX_M0) * c[:, 0]
        p1 = np.uint64(_PHILOX_M1) * c[:, 2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        c = np.stack([(hi1 ^ c[:, 1] ^ k0) & mask, lo1, (hi0 ^ c[:, 3] ^ k1) & mask, lo0], axis=1)
        k0 = (k0 + np.uint64(_PHILOX_W0)) & mask
        k1 = (k1 + np.uint64(_PHILOX_W1)) & mask
    return c.astype(np.uint32)


def gumbel_noise(seed: int, draw: int, vocab: int) -> np.ndarray:
    """Noise ``-log(-log(u))`` for every token of the vocabulary, for one request's draw number
    ``draw``: ``u`` from word 0 of ``philox(counter=(token, draw, 0, 0), key=(seed_lo, seed_hi))``,
    mapped to (0,1) as ``(x + 0.5) * 2**-32`` in float32."""
    ctr = np.zeros((vocab, 4), dtype=np.uint64)
    ctr[:, 0] = np.arange(vocab, dtype=np.uint64)
    ctr[:, 1] = np.uint64(draw)
    r = philox4x32(ctr, (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))[:, 0]
    u = (r.astype(np.float64) + 0.5) * (2.0 ** -32)
    u = np.minimum(u.astype(np.float32), np.float32(1.0 - 2.0 ** -24))
    return (-np.log(-np.log(u.astype(np.float32)))).astype(np.float32)


def apply_penalties(logits: np.ndarray, prev, rep: float, freq: float, pres: float) -> np.ndarray:
    """Repetition / frequency / presence penalties over earlier generated tokens
    (src/quanta/shim/omlx.py:344-363)."""
    if not len(prev) or (rep == 1.0 and freq == 0.0 and pres == 0.0):
        return logits
    counts = np.bincount(np.asarray(prev, dtype=np.int64), minlength=logits.shape[0]).astype(np.float32)
    seen = counts > 0
    out = logits.copy()
    if rep != 1.0:
        out = np.where(seen, np.where(out > 0, out / np.float32(rep), out * np.float32(rep)), out)
    return out - counts * np.float32(freq) - seen.astype(np.float32) * np.float32(pres)


def filter_logits(lg: np.ndarray, top_k: int, top_p: float, min_p: float) -> np.ndarray:
    """top-k (k-th largest threshold), then top-p (mass strictly before a token < p keeps it), then
    min-p (src/quanta/minimax/generate.py:34-53, 76-79).  ``lg`` is already divided by temperature."""
    lg = lg.astype(np.float32).copy()
    v = lg.shape[0]
    if 0 < top_k < v:
        kth = np.sort(lg)[v - top_k]
        lg[lg < kth] = -np.inf
    if 0.0 < top_p < 1.0:
        order = np.argsort(-lg, kind="stable")
        o = lg[order].astype(np.float64)
        p = np.exp(o - o.max())
        p /= p.sum()
        before = np.cumsum(p) - p
        keep = np.zeros(v, dtype=bool)
        keep[order] = before < top_p
        lg[~keep] = -np.inf
    if min_p > 0.0:
        p = np.exp(lg.astype(np.float64) - lg.max())
        p /= p.sum()
        lg[p < min_p * p.max()] = -np.inf
    return lg


def sample(logits, *, temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, seed=0, draw=0,
           prev=(), repetition_penalty=1.0, frequency_penalty=0.0, presence_penalty=0.0) -> int:
    """Greedy (first maximum) if ``temperature <= 0`` else a categorical draw over the filtered,
    tempered logits by the Gumbel-max rule with the counter-based noise above
    (src/quanta/minimax/generate.py:56-80)."""
    lg = np.asarray(logits, dtype=np.float32)
    lg = apply_penalties(lg, list(prev), repetition_penalty, frequency_penalty, presence_penalty)
    if temperature <= 0.0:
        return int(np.argmax(lg))
    lg = filter_logits(lg * np.float32(1.0 / temperature), top_k, top_p, min_p)
    return int(np.argmax(lg + gumbel_noise(seed, draw, lg.shape[0])))


def generate(weights, cfg, prompt, *, max_new_tokens, eos=(), act=None, compute=torch.float32,
             schedule=None, **sampling) -> list[int]:
    """Recompute the whole sequence for every new token (src/quanta/minimax/generate.py:92-148);
    an eos token ends the run and is not returned."""
    ids = list(prompt)
    out: list[int] = []
    for step in range(max_new_tokens):
        lg = forward_logits(weights, cfg, ids, act=act, compute=compute, schedule=schedule)[-1]
        tok = sample(lg.to(torch.float32).numpy(), draw=step, prev=out, **sampling)
        if tok in set(eos):
            break
        out.append(tok)
        ids.append(tok)
    return out
