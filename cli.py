"""Command line of the engine, in process (no server): generate from token ids or text.

Options follow the reference where it has them: `--model-path`, `--max-num-seqs`,
`--max-model-len`, `--max-prefill-len`, `--dtype {bf16,fp32}`, `--no-prewarm` are those of its
server (jllm/server.py:246-269); `--max-tokens` is its chat client's cap on new tokens
(cli.py:108); the line of statistics it prints per reply (tokens, tok/s, time to first token,
cli.py:184-192) is printed here per request.  Added: prompts as token ids, temperature,
seed, page options, and a random-weights mode for trying the engine without a checkpoint.

    python cli.py --model-path DIR --prompt-ids 1,2,3 --prompt-ids 7,8 --max-tokens 16
    python cli.py --random-weights 0 --config config.json --prompt-ids 5,17,3
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))


def parse_ids(text: str) -> list:
    return [int(t) for t in text.replace(",", " ").split()]


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("--model-path", default=os.environ.get("JLLM_MODEL_PATH"),
                   help="Path to HF model directory. Env: JLLM_MODEL_PATH.")
    p.add_argument("--max-num-seqs", type=int, default=4)
    p.add_argument("--max-model-len", type=int, default=2048)
    p.add_argument("--max-prefill-len", type=int, default=None,
                   help="longest prompt accepted (default: 512 as in the reference, or --max-model-len if that is less)")
    p.add_argument("--dtype", choices=["bf16", "fp32"], default="bf16")
    p.add_argument("--no-prewarm", dest="prewarm", action="store_false",
                   help="Skip the warm-up step at startup (kernels are then compiled and first run on the first request).")
    p.add_argument("--max-tokens", type=int, default=64, help="new tokens per prompt")
    p.add_argument("--prompt-ids", action="append", default=[], help="a prompt as token ids, e.g. 1,2,3 (repeatable)")
    p.add_argument("--prompt", action="append", default=[], help="a prompt as text (needs the folder's tokenizer)")
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--seed", type=int, default=None)
    p.add_argument("--eos-id", type=int, default=None)
    p.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    p.add_argument("--num-blocks", type=int, default=None, help="pages in the pool (default: worst case)")
    p.add_argument("--memory-fraction", type=float, default=None,
                   help="without --num-blocks: size the pool to this share of the free device memory")
    p.add_argument("--max-tokens-per-step", type=int, default=2048)
    p.add_argument("--ignore-eos", action="store_true", help="generate --max-tokens tokens whatever is sampled")
    p.add_argument("--no-prefix-cache", dest="prefix_cache", action="store_false")
    p.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                   help="do not read weights: draw them from this seed (needs --config or --model-path for config.json)")
    p.add_argument("--config", default=None, help="a config.json for --random-weights")
    args = p.parse_args(argv)

    from jax_vllm_b200 import (SamplingParams, add_request, has_work, load_from_path, make_driver, prewarm,
                               random_model, registry, step)

    if args.random_weights is not None:
        src = args.config or args.model_path
        if not src:
            p.error("--random-weights needs --config or --model-path")
        model = random_model(registry.config_from_path(src), args.random_weights, dtype=args.dtype)
        print(f"random weights (seed {args.random_weights}) for {src} ({args.dtype})", flush=True)
    else:
        if not args.model_path:
            p.error("--model-path is required")
        print(f"loading {args.model_path} ({args.dtype})...", flush=True)
        model = load_from_path(args.model_path, dtype=args.dtype)

    prompts = [parse_ids(t) for t in args.prompt_ids]
    tokenizer = None
    if args.prompt:
        try:
            from transformers import AutoTokenizer
            tokenizer = AutoTokenizer.from_pretrained(args.model_path)
        except Exception as exc:  # a tokenizer is optional: token ids are always accepted
            p.error(f"--prompt needs a tokenizer in --model-path ({exc}); use --prompt-ids")
        prompts += [tokenizer.encode(t) for t in args.prompt]
    if not prompts:
        p.error("give at least one --prompt-ids or --prompt")

    max_prefill_len = args.max_prefill_len if args.max_prefill_len is not None else min(512, args.max_model_len)
    driver = make_driver(model, max_num_seqs=args.max_num_seqs, max_model_len=args.max_model_len,
                         max_prefill_len=max_prefill_len, block_size=args.block_size, num_blocks=args.num_blocks,
                         max_tokens_per_step=args.max_tokens_per_step, prefix_cache=args.prefix_cache,
                         memory_fraction=args.memory_fraction)
    if args.prewarm:
        print(f"prewarm: done in {prewarm(driver):.1f}s", flush=True)

    sp = [SamplingParams(max_new_tokens=args.max_tokens, eos_id=args.eos_id, ignore_eos=args.ignore_eos,
                         temperature=args.temperature,
                         seed=None if args.seed is None else args.seed + i) for i in range(len(prompts))]
    t0 = time.perf_counter()
    ids = [add_request(driver, pr, s) for pr, s in zip(prompts, sp)]
    reqs = {i: driver.requests[i] for i in ids}
    while has_work(driver):
        step(driver)
    elapsed = time.perf_counter() - t0
    total = 0
    for i in ids:
        r = reqs[i]
        n = len(r.output_ids)
        total += n
        ttft = (r.first_token_time - r.arrival) if r.first_token_time else 0.0
        print(json.dumps({"request": i, "prompt_tokens": len(r.prompt_ids), "output_ids": r.output_ids}))
        if tokenizer is not None:
            print(tokenizer.decode(r.output_ids))
        print(f"  {n} tok · ttft {ttft:.3f}s", flush=True)
    st = driver.stats
    print(f"{total} tok · {total / elapsed:.1f} tok/s · {elapsed:.2f}s · steps {st.steps} · "
          f"prefix-hit tokens {st.cache_hit_tokens} · preemptions {st.preemptions} · "
          f"most pages in use {st.max_pages_in_use} of {st.pages_total} · most tokens in a step {st.max_step_tokens}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
