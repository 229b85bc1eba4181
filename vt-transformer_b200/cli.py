"""Command line of the engine.

    python -m vt_transformer_b200 generate --model DIR --prompt-ids 1,2,3 [--max-tokens N] ...
    python -m vt_transformer_b200 generate --model DIR --shell-mode
    python -m vt_transformer_b200 random-weights --config CONFIG.json --out DIR [--seed S] [--sigma X]

In vt-transformer's manner: its chat program takes token ids from a tokenizer, runs one step a
token, prints each token as it comes and ends a reply with "Generated N tokens, using S seconds"
(v1/models/qwen2-7b/chat.cpp:87-117); its front end's options are ``--model`` (alias of
``--tokenizer-path``/``--model-path``) and ``--shell-mode`` (sglfront/sglfront/server/args.py:94-189),
its request parameters temperature, top_k, top_p, ignore_eos, max_tokens
(sglfront/sglfront/core.py:6-13) with the shell's defaults from SGLFRONT_SHELL_* (max tokens 2048,
top_k -1, top_p 1.0, temperature 0.6: sglfront/sglfront/env.py:50-53), and its scheduler's settings
max_running_reqs, num_pages, max_seq_len, page_size, max_extend_tokens
(vt-transformer/core/vt_scheduler.hpp:33-38).  Text is outside this engine: prompts are token ids.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List


def _ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def _env(name: str, default, cast):
    v = os.environ.get("SGLFRONT_SHELL_" + name)
    return cast(v) if v is not None else default


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="vt_transformer_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate token ids for prompts of token ids")
    g.add_argument("--model", "--model-path", required=True, help="folder with config.json and model.safetensors")
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--device", default="cuda:0")
    g.add_argument("--fp32-weights", default="keep", choices=["keep", "round"],
                   help="matrices stored in 32-bit, with --dtype bfloat16: keep them (their products run the 32-bit "
                        "kernels) or round them to bfloat16 at load")
    g.add_argument("--prompt-ids", action="append", default=[], help="a prompt as token ids, e.g. 1,2,3 (repeatable)")
    g.add_argument("--prompt-file", help="a file with one prompt a line, as token ids")
    g.add_argument("--shell-mode", action="store_true", help="read prompts (token ids) line by line from standard input")
    g.add_argument("--max-tokens", type=int, default=_env("MAX_TOKENS", 2048, int))
    g.add_argument("--temperature", type=float, default=_env("TEMPERATURE", 0.6, float))
    g.add_argument("--top-k", type=int, default=_env("TOP_K", -1, int))
    g.add_argument("--top-p", type=float, default=_env("TOP_P", 1.0, float))
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--seed", type=int, default=0, help="seed of the requests' random numbers")
    g.add_argument("--max-running-reqs", type=int, default=128)
    g.add_argument("--num-pages", type=int, default=None)
    g.add_argument("--max-seq-len", type=int, default=4096)
    g.add_argument("--page-size", type=int, default=None, help="tokens in a page (default: the engine's, 64)")
    g.add_argument("--max-extend-tokens", type=int, default=8192, help="token budget of a step")
    g.add_argument("--chunk-size", type=int, default=None, help="longest portion of one prompt in a step")
    g.add_argument("--overlap", action="store_true",
                   help="enqueue the next decode step before the tokens of the one before are read")
    g.add_argument("--stats", action="store_true", help="print the scheduler's counters at the end")

    r = sub.add_parser("random-weights", help="write a model folder with seeded random weights")
    r.add_argument("--config", required=True, help="a config.json of a registered architecture")
    r.add_argument("--out", required=True, help="folder to write config.json and model.safetensors into")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--sigma", type=float, default=0.02)
    return ap


def _generate(args) -> int:
    from . import LLM, SamplingParams
    prompts = [_ids(p) for p in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [_ids(line) for line in f if line.strip()]
    if not prompts and not args.shell_mode:
        print("no prompt: give --prompt-ids, --prompt-file or --shell-mode", file=sys.stderr)
        return 2
    sizes = {} if args.page_size is None else {"page_size": args.page_size}
    llm = LLM(args.model, dtype=args.dtype, device=args.device, max_running_reqs=args.max_running_reqs,
              num_pages=args.num_pages, max_seq_len=args.max_seq_len,
              max_extend_tokens=args.max_extend_tokens, chunk_size=args.chunk_size, overlap=args.overlap,
              fp32_weights=args.fp32_weights, **sizes)
    params = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                            ignore_eos=args.ignore_eos, max_tokens=args.max_tokens, seed=args.seed)

    def reply(batch):
        t0 = time.time()
        outs = llm.generate(batch, params)
        dt = time.time() - t0
        for o in outs:
            print(" ".join(str(t) for t in o), flush=True)
        print(f"Generated {sum(len(o) for o in outs)} tokens, using {dt:.3f} seconds", file=sys.stderr, flush=True)

    if prompts:
        reply(prompts)
    if args.shell_mode:
        for line in sys.stdin:
            if line.strip():
                reply([_ids(line)])
    if args.stats:
        print(json.dumps(llm.stats), file=sys.stderr)
    return 0


def _random_weights(args) -> int:
    from .config import config_from_dict
    from .weights import write_random_model
    with open(args.config) as f:
        cfg = config_from_dict(json.load(f), args.config)
    write_random_model(cfg, args.out, seed=args.seed, sigma=args.sigma)
    print(args.out)
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    return _generate(args) if args.command == "generate" else _random_weights(args)


if __name__ == "__main__":
    sys.exit(main())
