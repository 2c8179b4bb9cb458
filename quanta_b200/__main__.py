"""Command line: ``python -m quanta_b200 <command>``.

    generate        tokens in, tokens out, options named as the reference's generate()
                    (src/quanta/minimax/generate.py:92-104): --max-new-tokens --temperature --top-k
                    --top-p --min-p --eos-id --seed, plus the engine's own.
    random-weights  write a model folder (config.json, model.safetensors) from a config file and a seed.
    build           compile the CUDA kernels now.

The reference has no module entry of its own for this model (its console script serves HTTP,
pyproject.toml:34-35); this one follows the manner of its ``python -m parity.<gate>`` scripts: plain
arguments, results on standard output, a non-zero exit on failure.
"""

from __future__ import annotations

import argparse
import json
import sys
import tempfile


def _ids(text: str) -> list[int]:
    return [int(x) for x in text.replace(",", " ").split()]


def _cmd_generate(a) -> int:
    from .config.registry import resolve
    from .engine.generate import LLM, generate
    from .engine.model import write_random_model
    model_dir = a.model
    tmp = None
    if model_dir is None:
        if a.random_weights is None or a.config is None:
            print("generate: give --model DIR, or --random-weights SEED with --config FILE", file=sys.stderr)
            return 2
        raw = json.loads(open(a.config).read())
        cfg = resolve(raw).config_cls.from_dict(raw)
        tmp = tempfile.TemporaryDirectory(prefix="quanta_b200_model_")
        model_dir = write_random_model(cfg, a.random_weights, tmp.name)
    prompts = []
    if a.prompt_ids:
        prompts.append(_ids(a.prompt_ids))
    if a.prompt_file:
        for line in open(a.prompt_file):
            if line.strip():
                prompts.append(_ids(line))
    if not prompts:
        print("generate: no prompt (use --prompt-ids \"1,2,3\" or --prompt-file FILE, one prompt a line)", file=sys.stderr)
        return 2
    llm = LLM(model_dir, dtype=a.dtype, device=a.device, page_size=a.block_size, num_pages=a.num_pages,
              max_requests=a.max_requests, max_step_tokens=a.max_step_tokens, prefill_chunk=a.prefill_chunk)
    eos = _ids(a.eos_id) if a.eos_id else None
    outs = generate(llm, prompts, max_new_tokens=a.max_new_tokens, temperature=a.temperature, top_k=a.top_k,
                    top_p=a.top_p, min_p=a.min_p, eos_id=eos, seed=a.seed,
                    repetition_penalty=a.repetition_penalty, frequency_penalty=a.frequency_penalty,
                    presence_penalty=a.presence_penalty)
    for out in outs:
        print(",".join(str(t) for t in out))
    if a.stats:
        print(json.dumps(llm.last_stats, default=str), file=sys.stderr)
    if tmp is not None:
        tmp.cleanup()
    return 0


def _cmd_random_weights(a) -> int:
    import torch
    from .config.registry import resolve
    from .engine.model import write_random_model
    raw = json.loads(open(a.config).read())
    cfg = resolve(raw).config_cls.from_dict(raw)
    out = write_random_model(cfg, a.seed, a.out, matrix_dtype=torch.float32 if a.store == "float32" else torch.bfloat16)
    print(out)
    return 0


def _cmd_build(a) -> int:
    from .csrc import build
    print(build.build(force=a.force))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m quanta_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="generate token ids after prompts")
    g.add_argument("--model", help="model folder (config.json + safetensors)")
    g.add_argument("--random-weights", type=int, metavar="SEED", help="use seeded random weights for --config")
    g.add_argument("--config", help="config.json for --random-weights")
    g.add_argument("--prompt-ids", help="token ids, comma or space separated")
    g.add_argument("--prompt-file", help="file with one prompt (token ids) a line")
    g.add_argument("--max-new-tokens", type=int, default=16)
    g.add_argument("--temperature", type=float, default=0.0, help="<= 0: greedy")
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--min-p", type=float, default=0.0)
    g.add_argument("--repetition-penalty", type=float, default=1.0)
    g.add_argument("--frequency-penalty", type=float, default=0.0)
    g.add_argument("--presence-penalty", type=float, default=0.0)
    g.add_argument("--eos-id", help="stop ids (default: the model's); comma separated")
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "bf16", "float32", "fp32"])
    g.add_argument("--device", default="cuda:0")
    g.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    g.add_argument("--num-pages", type=int, default=None, help="pages in the cache pool")
    g.add_argument("--max-step-tokens", type=int, default=4096, help="token budget of one step")
    g.add_argument("--prefill-chunk", type=int, default=4096, help="largest prompt portion (chunk_tokens of the reference's chunked prefill)")
    g.add_argument("--max-requests", type=int, default=64, help="requests live at a time")
    g.add_argument("--stats", action="store_true", help="print run statistics to standard error")
    g.set_defaults(fn=_cmd_generate)
    r = sub.add_parser("random-weights", help="write a model folder with seeded random weights")
    r.add_argument("--config", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--store", default="bfloat16", choices=["bfloat16", "float32"], help="dtype matrices are stored in")
    r.set_defaults(fn=_cmd_random_weights)
    b = sub.add_parser("build", help="compile the CUDA kernels")
    b.add_argument("--force", action="store_true")
    b.set_defaults(fn=_cmd_build)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
