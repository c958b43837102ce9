"""Trace replay: given token ids fed step by step through the engine's own model, step
function, cache and kernels; logits written to disk; nothing sampled.

A step is one JSON object: {"step": s, "entries": [{"id": r, "tokens": [...], "want":
[...]}, ...], "end": [r, ...]}.  All entries of a step form one batch.  A request is
admitted when its id first appears and keeps its pages until an `end` names it.  For a
step with wanted places the logits are written to `<out>/<step>.f32` as little-endian
float32 [wanted, vocab], in the order of the entries and of their `want`.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

from ..cache import CacheManager
from .batch import StepEntry
from .loading import load_from_path
from .runner import Runner

MAX_LIVE = 8


class Replayer:
    def __init__(self, model_dir, dtype, out_dir, max_tokens: int, page_size: int = 16, device="cuda:0"):
        self.out = Path(out_dir)
        self.out.mkdir(parents=True, exist_ok=True)
        self.model = load_from_path(model_dir, dtype=dtype, device=device)
        num_pages = max(1, -(-int(max_tokens) // page_size))
        self.cache = CacheManager(self.model.cache_needs(), page_size, num_pages, MAX_LIVE, prefix_cache=False)
        self.runner = Runner(self.model, self.cache, device, self.model.ctx.dtype)

    def run_step(self, record: dict) -> None:
        step = record["step"]
        entries = []
        for e in record.get("entries", []):
            rid, tokens = e["id"], [int(t) for t in e["tokens"]]
            if not tokens:
                raise ValueError(f"step {step}: request {rid!r} brings no tokens")
            rc = self.cache.live.get(rid) or self.cache.admit(rid)
            entries.append(StepEntry(rc, tokens, tuple(int(w) for w in e.get("want", ()))))
        if len({id(e.cache) for e in entries}) != len(entries):
            raise ValueError(f"step {step}: a request appears twice")
        logits = self.runner.run(entries)
        host = logits.to("cpu")            # also waits for the step
        self.runner.check_kernels()
        if host.shape[0]:
            arr = host.numpy().astype("<f4", copy=False)
            tmp = self.out / f".{step}.f32.tmp"
            arr.tofile(tmp)
            tmp.replace(self.out / f"{step}.f32")
        for rid in record.get("end", []):
            if rid in self.cache.live:
                self.cache.release(rid)

    def run_stream(self, lines, done=sys.stdout) -> None:
        for line in lines:
            line = line.strip()
            if not line:
                continue
            record = json.loads(line)
            self.run_step(record)
            print(f"done {record['step']}", file=done, flush=True)


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64); sizes the cache pool")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page (a divisor of 64)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if 64 % args.page_size:
        ap.error("--page-size must divide 64")
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; this engine has no CPU path", file=sys.stderr)
        return 3
    print(f"[trace_run] loading {args.model} as {args.dtype}; kernels are compiled at the first call",
          file=sys.stderr, flush=True)
    rep = Replayer(args.model, args.dtype, args.out, args.max_tokens, args.page_size, args.device)
    print("[trace_run] ready", file=sys.stderr, flush=True)
    rep.run_stream(sys.stdin)
    return 0
