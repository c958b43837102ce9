"""Trace replay: given token ids fed step by step through the engine's own model, step
function, cache and kernels; logits written to disk; nothing sampled.

A step is one JSON object: {"step": s, "entries": [{"id": r, "tokens": [...], "want":
[...]}, ...], "end": [r, ...]}.  All entries of a step form one batch.  A request is
admitted when its id first appears and keeps its pages until an `end` names it.  For a
step with wanted places the logits are written to `<out>/<step>.f32` as little-endian
float32 [wanted, vocab], in the order of the entries and of their `want`.  Beside it,
`<out>/<step>.json` says what the step did to the cache and what the batch was made of:
pages allocated and given back, tokens taken from pages that an earlier request had
filled (prefix reuse), pages free afterwards, entries of one token and tiles per class of
the attention's work lists, and whether the step was replayed from a CUDA graph.

Two switches make a trace run what generation runs: `prefix_cache` lets a new request take
the pages of a known prefix of its first portion, up to its first wanted place (the
logits of a place that is taken from the cache are not computed, so reuse never reaches
a wanted place; generation wants the last place only, jllm/engine/cache.py:33-46 has the
reference's lookup); `cuda_graphs` replays steps of single tokens from a captured graph,
as the entry point does by default.
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
    def __init__(self, model_dir, dtype, out_dir, max_tokens: int, page_size: int = 16, device="cuda:0",
                 prefix_cache: bool = False, cuda_graphs: bool = False):
        self.out = Path(out_dir)
        self.out.mkdir(parents=True, exist_ok=True)
        self.model = load_from_path(model_dir, dtype=dtype, device=device)
        num_pages = max(1, -(-int(max_tokens) // page_size))
        self.cache = CacheManager(self.model.cache_needs(), page_size, num_pages, MAX_LIVE, prefix_cache=prefix_cache)
        self.runner = Runner(self.model, self.cache, device, self.model.ctx.dtype,
                             max_model_len=num_pages * page_size, cuda_graphs=cuda_graphs)
        self.records: list = []            # the metadata of every step run so far

    def _admit(self, rid, tokens, want):
        """A new request: with prefix reuse it may take pages that hold the start of its first portion, short
        of the first place whose logits are wanted and of the portion's last token."""
        upto = min([len(tokens) - 1] + [w for w in want])
        return self.cache.admit(rid, tokens[:upto + 1])

    def run_step(self, record: dict) -> dict:
        step = record["step"]
        entries = []
        before = dict(self.cache.stats)
        for e in record.get("entries", []):
            rid, tokens = e["id"], [int(t) for t in e["tokens"]]
            want = tuple(int(w) for w in e.get("want", ()))
            if not tokens:
                raise ValueError(f"step {step}: request {rid!r} brings no tokens")
            if any(not 0 <= w < len(tokens) for w in want):
                raise ValueError(f"step {step}: request {rid!r} wants a place outside its {len(tokens)} tokens")
            rc = self.cache.live.get(rid)
            skip = 0
            if rc is None:
                rc = self._admit(rid, tokens, want)
                skip = rc.num_tokens                      # tokens found in the cache: not run again
            entries.append(StepEntry(rc, tokens[skip:], tuple(w - skip for w in want)))
        if len({id(e.cache) for e in entries}) != len(entries):
            raise ValueError(f"step {step}: a request appears twice")
        graphs_before = self.runner.graph_replays
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
        after = self.cache.stats
        tiles = {}
        for cls in self.runner.builder.tile_token_sizes:
            n = sum(-(-len(e.tokens) // cls[0]) for e in entries if len(e.tokens) > 1 and cls[1] <= len(e.tokens) < cls[2])
            tiles[f"{cls[0]} tokens, entries of {cls[1]} or more"] = n
        meta = {"step": step, "tokens": sum(len(e.tokens) for e in entries), "entries": len(entries),
                "single_token_entries": sum(1 for e in entries if len(e.tokens) == 1), "tiles": tiles,
                "pages_allocated": after["pages_allocated"] - before["pages_allocated"],
                "pages_released": after["pages_released"] - before["pages_released"],
                "prefix_hit_tokens": after["prefix_hit_tokens"] - before["prefix_hit_tokens"],
                "prefix_hit_pages": after["prefix_hit_pages"] - before["prefix_hit_pages"],
                "pages_free": [g.pool.num_free for g in self.cache.groups],
                "live_requests": len(self.cache.live),
                "replayed_graph": self.runner.graph_replays > graphs_before}
        (self.out / f"{step}.json").write_text(json.dumps(meta))
        self.records.append(meta)
        return meta

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
    ap.add_argument("--out", required=True, help="folder for <step>.f32 (logits) and <step>.json (what the step did)")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64); sizes the cache pool")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page (a divisor of 64)")
    ap.add_argument("--prefix-cache", action="store_true",
                    help="a new request takes pages that hold the start of its first portion, short of its first wanted place")
    ap.add_argument("--cuda-graphs", action="store_true",
                    help="steps of single tokens are replayed from a captured graph, as in generation")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if 64 % args.page_size:
        ap.error("--page-size must divide 64")
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; this engine has no CPU path", file=sys.stderr)
        return 3
    print(f"[trace_run] loading {args.model} as {args.dtype}; kernels are compiled at the first call",
          file=sys.stderr, flush=True)
    rep = Replayer(args.model, args.dtype, args.out, args.max_tokens, args.page_size, args.device,
                   prefix_cache=args.prefix_cache, cuda_graphs=args.cuda_graphs)
    print("[trace_run] ready", file=sys.stderr, flush=True)
    rep.run_stream(sys.stdin)
    return 0
