#!/usr/bin/env python3
"""Benchmark: decode tokens a second of the MiniMax-M3 engine at the M2-family layer sizes.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on standard output.  A "step" is one decode step of the whole batch.  The default run
has the layer sizes of the baseline's third configuration (hidden 3072, 48 q / 8 kv heads of 128,
rotary 64, 256 experts top-8 of width 1536, vocabulary 200064) with seeded random weights, 16 of the
model's 62 layers (about 120 GB of bfloat16 weights), a batch of 8 requests that have each read a
2,048-token prompt and then decode 256 steps (the default K), and a cache sized for the 4,096-token
context.

* ``value``: decoded tokens a second, timed on the device with CUDA events around every step (the
  step function and the sampling kernel), after warm-up steps.  Each step reads tens of GB of
  weights, far more than the 126 MB L2, so no flush is needed between steps (said in ``config``).
* ``e2e``: the same through the Python entry point (``LLM``): host token ids in, sampled ids out,
  every step with its pinned host->device copy of the step's integers and device->host read of
  the sampled ids.
* ``prefill``: one 2,048-token prompt as one step: tokens a second, and flops / time / tensor peak
  (``frac``); the step reads all 256 experts of every layer for 64 rows each, so it is bound by memory:
  ``hbm_frac`` is its weight bytes / time / copy bandwidth.
* ``roofline``: bytes the decode step has to read (each weight it uses once, counted from the
  experts the router really chose, plus the cache of the live requests) / time / copy bandwidth.
* ``points``: decode at batch 1 and 64 (``decode_b1``, ``decode_b64``: tokens a second over at least 32
  timed steps), each with its time a step, the bytes the step has to read counted from the experts its
  router chose and the requests' contexts, that over time over copy bandwidth (``_frac``) and the same
  through the Python entry point (``_e2e``); and one step of 8 prompts of 2,048 tokens
  (``prefill_16384``), which is bound by the tensor cores: its flops / time over the sustained tensor peak.
Peaks are read from MEASURED_PEAKS.json beside this file when it is there, else the stated fallback.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FULL_LAYERS = 62
PREFILL_TOKENS = 2048
SIZES = dict(vocab_size=200064, hidden_size=3072, intermediate_size=1536, num_attention_heads=48,
             num_key_value_heads=8, head_dim=128, rotary_dim=64, rope_theta=5e6, use_qk_norm=True,
             qk_norm_type="per_layer", num_local_experts=256, num_experts_per_tok=8, use_routing_bias=True,
             rms_norm_eps=1e-6, tie_word_embeddings=False, architectures=["MiniMaxM3ForCausalLM"],
             model_type="minimax_m3")
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            raw = json.loads(p.read_text())
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(raw.get(k), (int, float)):
                    out[k] = float(raw[k])
            return out, "measured"
        except (ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def prefill_flops(c, layers: int, T: int) -> float:
    H, hd, nq, nkv = c["hidden_size"], c["head_dim"], c["num_attention_heads"], c["num_key_value_heads"]
    proj = 2 * T * H * (nq + 2 * nkv) * hd + 2 * T * nq * hd * H
    attn = 2 * 2 * nq * hd * T * (T + 1) / 2
    router = 2 * T * H * c["num_local_experts"]
    experts = 2 * T * c["num_experts_per_tok"] * 3 * H * c["intermediate_size"]
    return layers * (proj + attn + router + experts) + 2 * H * c["vocab_size"]


def decode_bytes(model, c, layers: int, ctx_tokens: list[int], distinct_experts: list[int]) -> float:
    """Bytes one decode step has to read: every weight it uses once + the cache of the live requests."""
    H, hd, nq, nkv, I = c["hidden_size"], c["head_dim"], c["num_attention_heads"], c["num_key_value_heads"], c["intermediate_size"]
    attn_w = 2 * (H * (nq + 2 * nkv) * hd + nq * hd * H)
    router_w = 4 * c["num_local_experts"] * H
    expert_w = 2 * 3 * H * I
    kv = sum(ctx_tokens) * 2 * nkv * hd * 2
    per_layer_fixed = attn_w + router_w + kv
    head = 2 * H * c["vocab_size"]
    return layers * per_layer_fixed + expert_w * sum(distinct_experts) + head


def run_ours(args) -> dict:
    import torch
    from quanta_b200 import kernels
    from quanta_b200.config import MiniMaxM3Config
    from quanta_b200.engine.generate import LLM
    from quanta_b200.engine.model import random_model
    from quanta_b200.engine.scheduler import Request, SamplingParams
    from quanta_b200.engine.step import StepEntry
    from quanta_b200.parts.moe import SigmoidTopKExperts
    import random

    pk, pk_src = peaks()
    layers, B, prompt_len, context = args.layers, args.batch, args.prompt_len, args.context
    raw = dict(SIZES, num_hidden_layers=layers)
    cfg = MiniMaxM3Config.from_dict(raw)
    t0 = time.time()
    model = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    torch.cuda.synchronize()
    weights_gb = round(torch.cuda.memory_allocated() / 1e9, 1)
    print(f"[bench] model of {layers} layers built in {time.time() - t0:.0f} s, "
          f"{torch.cuda.memory_allocated() / 1e9:.1f} GB on the device", file=sys.stderr, flush=True)
    page = 16
    max_b = max([B] + ([1, 64] if args.points else []))
    llm = LLM(model, page_size=page, num_pages=max_b * context // page, max_requests=max_b,
              max_step_tokens=max(prompt_len, max_b), prefill_chunk=prompt_len, max_position=context)
    eng = llm.engine
    rng = random.Random(0)
    V = cfg.vocab_size

    def toks(n):
        return [rng.randrange(V) for _ in range(n)]

    greedy_out = torch.empty(64, dtype=torch.int32, device="cuda:0")

    def timed_steps(make_entries, n_warm, n_timed, sample_rows):
        """Device time of each of n_timed steps (ms)."""
        evs = []
        for i in range(n_warm + n_timed):
            entries = make_entries(i)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            lg = eng.step(entries)
            if sample_rows:
                kernels.sample_rows(lg, None, None, greedy_out[: lg.shape[0]])
            b.record()
            evs.append((a, b))
        torch.cuda.synchronize()
        eng.check()
        return [a.elapsed_time(b) for a, b in evs[n_warm:]]

    # ---- prefill: one 2,048-token prompt as one step ----
    pf_tokens = min(PREFILL_TOKENS, prompt_len)
    pre_ms = []
    for i in range(3 + 3):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p = toks(pf_tokens)
        torch.cuda.synchronize()
        a.record()
        eng.step([StepEntry(("pf", i), p, (pf_tokens - 1,))], end=[("pf", i)])
        b.record()
        torch.cuda.synchronize()
        pre_ms.append(a.elapsed_time(b))
    pre = statistics.median(pre_ms[3:])
    pf = prefill_flops(raw, layers, pf_tokens)
    # the step reads every expert once: its bytes / time / copy bandwidth says how close to ITS bound it runs
    pf_bytes = decode_bytes(model, raw, layers, [], [cfg.num_local_experts] * layers)
    prefill = {"value": round(pf_tokens / pre * 1e3, 1), "tokens": pf_tokens, "ms": round(pre, 3),
               "frac": round(pf / (pre * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               "hbm_frac": round(pf_bytes / (pre * 1e-3) / (pk["hbm_gbs"] * 1e9), 4)}
    print(f"[bench] prefill {prefill}", file=sys.stderr, flush=True)

    # ---- decode, device-timed ----
    def decode_run(batch, n_warm, n_timed):
        rids = [("d", batch, i) for i in range(batch)]
        for rid in rids:
            prompt = toks(prompt_len)
            for lo in range(0, prompt_len, args.prefill_chunk or prompt_len):      # whole, or in portions
                eng.step([StepEntry(rid, prompt[lo: lo + (args.prefill_chunk or prompt_len)], ())])
        kernels.LAUNCHES = 0
        ms = timed_steps(lambda i: [StepEntry(rid, [rng.randrange(V)], (0,)) for rid in rids], n_warm, n_timed, True)
        launches = kernels.LAUNCHES * n_timed // (n_warm + n_timed)
        ctx = [eng.manager.length(rid) - n_timed // 2 for rid in rids]      # keys a request has in the middle timed step
        distinct = []
        for blk in model.blocks:
            ff = blk.feed_forward
            if isinstance(ff, SigmoidTopKExperts) and ff.last_counts is not None:
                distinct.append(int((ff.last_counts > 0).sum()))
        for rid in rids:
            eng.release(rid)
        return ms, launches, ctx, distinct

    clocks = ClockSampler()
    clocks.start()
    ms, launches, ctx, distinct = decode_run(B, args.warmup, args.steps)
    clock_info = clocks.stop()
    step_ms = statistics.fmean(ms)
    value = B / step_ms * 1e3
    need = decode_bytes(model, raw, layers, ctx, distinct)
    achieved = need / (step_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(need), "peaks": pk_src}
    print(f"[bench] decode b{B}: {value:.1f} tok/s, {step_ms:.3f} ms/step, roofline {roofline}", file=sys.stderr, flush=True)

    def e2e_run(batch, n_timed):
        """Decode tokens a second through ``LLM.run``: host ids in, sampled ids out, every step."""
        n_new = args.warmup + n_timed + 1 + 8          # the prompts enter a few at a time: later ones decode fewer pure steps
        chunk = args.prefill_chunk or prompt_len
        llm.sched_opts["max_step_tokens"] = min(batch, 8) * chunk     # prompts advance together, then pure decode steps
        llm.sched_opts["prefill_chunk"] = chunk
        reqs = [Request(rid=("e", batch, i), prompt=toks(prompt_len), params=SamplingParams(max_new_tokens=n_new))
                for i in range(batch)]
        llm.run(reqs)
        dec = [s for s in llm.step_log if s["tokens"] == s["sampled"] == batch][args.warmup:]
        val = batch * (len(dec) - 1) / (dec[-1]["t_end"] - dec[0]["t_end"]) if len(dec) >= 2 else None
        return val, (dec[-1] if dec else None)

    points = {}
    if args.points:
        for b in (1, 64):
            n_timed = max(32, args.steps // 4)
            pms, _, pctx, pdistinct = decode_run(b, 3, n_timed)
            p_ms = statistics.fmean(pms)
            p_bytes = decode_bytes(model, raw, layers, pctx, pdistinct)
            key = f"decode_b{b}"
            points[key] = round(b / p_ms * 1e3, 1)
            points[key + "_ms"] = round(p_ms, 4)
            points[key + "_steps"] = n_timed
            points[key + "_bytes"] = int(p_bytes)
            points[key + "_experts_read"] = int(sum(pdistinct))
            points[key + "_frac"] = round(p_bytes / (p_ms * 1e-3) / (pk["hbm_gbs"] * 1e9), 4)
            if args.e2e:
                val, _ = e2e_run(b, n_timed)
                points[key + "_e2e"] = round(val, 1) if val else None
            print(f"[bench] decode b{b}: {points[key]} tok/s, {p_ms:.3f} ms/step, {points[key + '_frac']} of the copy "
                  f"bandwidth, e2e {points.get(key + '_e2e')}", file=sys.stderr, flush=True)
        # one step of 8 prompts of 2,048 tokens: 64 x 8 rows an expert on average, bound by the tensor cores
        big, big_ms = 8, []
        for i in range(2 + 3):
            a, bb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            entries = [StepEntry(("pb", i, j), toks(pf_tokens), (pf_tokens - 1,)) for j in range(big)]
            torch.cuda.synchronize()
            a.record()
            eng.step(entries, end=[e.rid for e in entries])
            bb.record()
            torch.cuda.synchronize()
            big_ms.append(a.elapsed_time(bb))
        bm_ = statistics.median(big_ms[2:])
        big_flops = big * (pf - 2 * cfg.hidden_size * cfg.vocab_size) + big * 2 * cfg.hidden_size * cfg.vocab_size
        points["prefill_16384"] = round(big * pf_tokens / bm_ * 1e3, 1)
        points["prefill_16384_ms"] = round(bm_, 3)
        points["prefill_16384_frac_sustained"] = round(big_flops / (bm_ * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
        print(f"[bench] prefill of {big} x {pf_tokens} tokens in one step: {bm_:.2f} ms, "
              f"{points['prefill_16384_frac_sustained']} of the sustained tensor peak", file=sys.stderr, flush=True)

    # ---- end to end through the Python entry point ----
    e2e_val, last = e2e_run(B, args.steps) if args.e2e else (None, None)
    e2e = {"value": round(e2e_val, 1) if e2e_val else None, "unit": "tokens/s",
           "h2d_bytes_per_step": last["h2d_bytes"] if last else None,
           "d2h_bytes_per_step": last["d2h_bytes"] if last else None}

    config = {"model": "MiniMax-M3 (M2-family sizes), random weights", "weights_gb": weights_gb, "layers": layers, "layers_full": FULL_LAYERS,
              "hidden": 3072, "q_heads": 48, "kv_heads": 8, "head_dim": 128, "rotary_dim": 64, "experts": 256,
              "top_k": 8, "expert_width": 1536, "vocab": 200064, "global_batch": B, "seq_len": context,
              "prompt_len": prompt_len, "kv_block": page, "parallelism": "single GPU",
              "l2": "no flush: each step reads >20 GB of weights, inputs larger than L2"}
    return {"metric": f"decode tokens/s (batch {B}, {prompt_len}-token prompts, context {context})", "value": round(value, 1),
            "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(step_ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (seeded uniform token ids, seeded random weights)",
            "config": config, "prefill": prefill, "roofline": roofline, "points": points, "e2e": e2e,
            "gpu_launches": int(launches), "clocks": clock_info, "impl": "ours"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=16, help="layers built (the model has 62)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--prefill-chunk", type=int, default=0,
                    help="feed the prompts of the decode runs in portions of this many tokens (0: whole)")
    ap.add_argument("--no-e2e", dest="e2e", action="store_false", help="skip the run through the Python entry point")
    ap.add_argument("--no-points", dest="points", action="store_false", help="skip the batch 1 and 64 points")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "pmrjge/quanta runs on Apple MLX only (mlx is not installable here; its build backend "
                          "uv_build is absent too), it has no CUDA path"}))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.prompt_len + args.warmup + args.steps + 1 > args.context:
        ap.error(f"--context {args.context} is too short for prompts of {args.prompt_len} tokens and "
                 f"{args.warmup} + {args.steps} + 1 decoded tokens")
    out = run_ours(args)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
