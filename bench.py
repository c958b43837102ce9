"""Decode and prefill throughput of the engine on one B200, for the Qwen3-8B shape with
random bfloat16 weights: the reference's headline metric (decoded tokens per second) at its largest
dense Qwen3 configuration.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]
    python bench.py --workload mixed14b|long32b      # a serving workload of a larger shape (its own JSON line)

Prints ONE JSON line.  `value` is decoded tokens per second at the given batch, each request
holding 2,048 tokens of context, timed on the device with CUDA events over K decode steps
after W warm-up steps (a "step" is one decode step: one token for every request of the
batch).  `e2e` is the same through the Python entry point (`add_request`/`step`), token ids
from the host and sampled tokens back to the host in every step.  `prefill` is one
2,048-token prompt in one step; `points` holds decoding at batch 1 and 64; `roofline` is
the decode step's bytes (every weight it uses once, and the cache of the live requests)
over its time, against the measured copy bandwidth.  Weights (15 GB) are far larger than
the L2, so nothing is flushed between iterations.  The engine runs on one GPU only: for
--gpus N > 1 it says so and exits with 2.
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], vocab_size=151936, hidden_size=4096, intermediate_size=12288,
                num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=40960, tie_word_embeddings=False)
CONTEXT = 2048
PREFILL_TOKENS = 2048
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"]))}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.proc = None
        self.index = index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.summary = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        mhz, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                mhz.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if mhz:
            self.summary = {"sm_mhz": statistics.median(mhz), "sm_max_mhz": max(mx), "reasons": sorted(reasons)}


def layer_params(c):
    H, I, D = c["hidden_size"], c["intermediate_size"], c["head_dim"]
    Hq, Hkv = c["num_attention_heads"], c["num_key_value_heads"]
    return H * (Hq + 2 * Hkv) * D + Hq * D * H + 3 * H * I


def decode_bytes(c, layers, batch, ctx, itemsize=2):
    weights = (layers * layer_params(c) + c["vocab_size"] * c["hidden_size"]) * itemsize
    kv = batch * ctx * layers * 2 * c["num_key_value_heads"] * c["head_dim"] * itemsize
    return weights + kv


def prefill_flops(c, layers, T):
    gemm = 2 * T * layers * layer_params(c) + 2 * c["vocab_size"] * c["hidden_size"]
    attn = layers * 4 * c["num_attention_heads"] * c["head_dim"] * T * (T + 1) // 2
    return gemm + attn


def fake_context(driver, batch, ctx):
    """`batch` live requests that hold `ctx` tokens each, their pages filled with random keys and values
    (what the tokens were does not change the work of a decode step)."""
    import torch
    rcs = []
    for i in range(batch):
        rc = driver.cache.admit(("bench", i))
        driver.cache.grow(rc, ctx)
        rc.num_tokens = ctx
        rcs.append(rc)
    for grp in driver.cache.groups:
        grp.k.normal_(0, 1)
        grp.v.normal_(0, 1)
    torch.cuda.synchronize()
    return rcs


MIN_TIMED_SECONDS = 0.5      # a timed region shorter than this is repeated until it adds up to it
MAX_CONTEXT = 4096            # requests of the decode runs never grow beyond this


def time_decode(model, batch, steps, warmup, ctx=CONTEXT):
    """Device time of `steps` decode steps at `batch`, repeated until MIN_TIMED_SECONDS are timed (at most until the
    requests reach MAX_CONTEXT tokens); returns (median ms per step over the repeats, launches per step, repeats,
    all the repeats' ms per step)."""
    import torch
    from jax_vllm_b200 import make_driver, ops
    from jax_vllm_b200.engine import StepEntry
    max_len = MAX_CONTEXT
    driver = make_driver(model, max_num_seqs=batch, max_model_len=max_len, block_size=PAGE, prefix_cache=False)
    rcs = fake_context(driver, batch, ctx)
    runner, cache, sampler = driver.runner, driver.cache, driver.sampler

    def one(i):
        entries = []
        for b, rc in enumerate(rcs):
            cache.grow(rc, rc.num_tokens + 1)
            entries.append(StepEntry(rc, [(i * 7919 + b) % 1000], (0,)))
        logits = runner.step(entries)
        toks = sampler.greedy(logits)
        for e in entries:
            rc = e.cache
            rc.num_tokens += 1
        return toks

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    per_step, launches, done = [], 0, warmup
    most = max(1, (MAX_CONTEXT - ctx - warmup - 1) // steps)
    while True:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        before = ops.launch_count
        start.record()
        for i in range(steps):
            one(done + i)
        end.record()
        torch.cuda.synchronize()
        done += steps
        per_step.append(start.elapsed_time(end) / steps)
        launches = (ops.launch_count - before) // steps
        if sum(per_step) * steps >= MIN_TIMED_SECONDS * 1e3 or len(per_step) >= most:
            break
    runner.check_kernels()
    del driver, runner, cache
    torch.cuda.empty_cache()
    return statistics.median(per_step), launches, len(per_step), per_step


def time_prefill(model, tokens, warmup, reps=3):
    import torch
    from jax_vllm_b200 import make_driver
    from jax_vllm_b200.engine import StepEntry
    max_len = -(-(tokens + 16) // PAGE) * PAGE
    driver = make_driver(model, max_num_seqs=1, max_model_len=max_len, block_size=PAGE, prefix_cache=False,
                         max_tokens_per_step=tokens)
    ids = [(i * 7919 + 13) % 1000 for i in range(tokens)]
    times = []
    for r in range(warmup + reps):
        rc = driver.cache.admit(("prefill", r))
        driver.cache.grow(rc, tokens)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        driver.runner.step([StepEntry(rc, ids, (tokens - 1,))])
        e.record()
        torch.cuda.synchronize()
        if r >= warmup:
            times.append(s.elapsed_time(e))
        driver.cache.release(("prefill", r))
    driver.runner.check_kernels()
    del driver
    torch.cuda.empty_cache()
    return statistics.median(times)


def time_e2e(model, batch, steps, warmup, ctx=CONTEXT):
    """Through the entry point: `batch` prompts of `ctx` tokens from the host, then decode steps whose
    sampled tokens come back to the host each step."""
    import torch
    from jax_vllm_b200 import SamplingParams, add_request, make_driver, step
    runs = max(3, min(25, int(MIN_TIMED_SECONDS / (steps * 0.004)) + 1))
    new = min(warmup + runs * steps + 4, MAX_CONTEXT - ctx)
    runs = max(1, (new - warmup - 4) // steps)
    max_len = -(-(ctx + new) // PAGE) * PAGE
    driver = make_driver(model, max_num_seqs=batch, max_model_len=max_len, block_size=PAGE, prefix_cache=False,
                         max_tokens_per_step=max(2048, batch))
    for b in range(batch):
        add_request(driver, [(i * 31 + b * 977) % 50000 for i in range(ctx)], SamplingParams(max_new_tokens=new))
    while any(len(r.output_ids) < 1 + warmup for r in driver.requests.values()):   # prompts, then warm-up decodes
        step(driver)
    # `runs` runs of `steps` steps (a run is tens of milliseconds of wall clock on a shared host, where one hiccup of
    # the host halves it): the median counts, the fastest is given beside it
    rates = []
    for _ in range(runs):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        emitted = 0
        for _ in range(steps):
            emitted += len(step(driver))
        torch.cuda.synchronize()
        rates.append(emitted / (time.perf_counter() - t0))
    # one copy per step: the batch description (tokens, positions, block tables, work lists) and, behind it in
    # the same buffer, seeds, counters and temperatures of the sampler
    g = driver.runner.graphs_sampled.get(batch)
    if g is not None:
        h2d = g.total * 4
    else:
        g = driver.runner.graphs.get(batch)
        h2d = (g.layout.total * 4 if g is not None else 0) + batch * (4 + 16)
    d2h = (batch + 1) * 4                        # sampled tokens and the kernels' status word
    del driver
    torch.cuda.empty_cache()
    return statistics.median(rates), max(rates), len(rates), h2d, d2h


def micro(spec: str, reps: int, eager: bool = False) -> int:
    """One kernel alone on data larger than the L2, for profiling:
    gemm:<N>x<K>:<M>:<impl>  the prompt product, impl = tcgen05 | tcgen05_swiglu | library (cuBLAS)
    linear:<N>x<K>:<M>[:parts][:stream|:skinny|:library]   the decode product of M rows with an [N, K] weight (several weights in turn):
                         as the engine picks it, or the tcgen05 kernel, the mma.sync kernel, cuBLAS
    attn_decode:<B>:<CTX>[:<SPLIT>[:<PAGE>[:<KV HEADS>[:<QUERY HEADS PER KV HEAD>]]]]   split decode attention of B requests with CTX cached tokens (8B head layout,
                         several caches in turn so that none stays in the L2), mma.sync kernel
    attn_decode_tcgen05:<B>:<CTX>[:<SPLIT>[:<PAGE>]]   the same with the tcgen05 kernel
    (the decode kernels are timed as replays of a CUDA graph of one launch per cache, as the engine runs them)
    attn_prefill:<T>     prompt attention of one request of T tokens (8B head layout), mma.sync kernel
    attn_prefill_tcgen05:<T>[:<PAGE>]   the same with the tcgen05 kernel"""
    import torch
    from jax_vllm_b200 import ops
    kind, *rest = spec.split(":")
    dev = "cuda:0"
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if kind == "gemm":           # gemm:<N>x<K>:<M>:<impl>  impl = tcgen05 | tcgen05_swiglu | library
        n, k = (int(v) for v in rest[0].split("x"))
        m, impl = int(rest[1]), rest[2]
        copies = max(2, int(300e6 // (n * k * 2)) + 1)
        ws = [(torch.randn(n, k, device=dev) * 0.02).to(torch.bfloat16) for _ in range(copies)]
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        if impl == "library":
            run = lambda i: torch.mm(x, ws[i % copies].t())
        else:
            run = lambda i: ops.gemm_tcgen05(x, ws[i % copies], "swiglu" if impl.endswith("swiglu") else "bf16")
        for i in range(3):
            run(i)
        torch.cuda.synchronize()
        start.record()
        for i in range(reps):
            run(i)
        end.record()
        torch.cuda.synchronize()
        us = start.elapsed_time(end) / reps * 1e3
        print(json.dumps({"micro": spec, "us": round(us, 2), "TFLOP/s": round(2.0 * m * n * k / us / 1e6, 1)}))
        return 0
    if kind == "linear":
        n, k = (int(v) for v in rest[0].split("x"))
        m = int(rest[1])
        copies = max(2, int(400e6 // (n * k * 2)) + 1)
        ws = [(torch.randn(n, k, device=dev) * 0.02).to(torch.bfloat16) for _ in range(copies)]
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        parts_ok = "parts" in rest[2:]        # let the kernel cut k and leave the parts of a sum
        if "skinny" in rest[2:]:              # the mma.sync kernel, whatever the dispatcher would take
            run = lambda i: ops.linear_skinny(x, ws[i % copies], torch.bfloat16, parts_ok)
        elif "stream" in rest[2:]:            # the tcgen05 product for larger batches, whatever the rows
            run = lambda i: ops.linear_stream(x, ws[i % copies], torch.bfloat16, parts_ok)
        elif "library" in rest[2:]:
            run = lambda i: torch.mm(x, ws[i % copies].t())
        else:
            run = lambda i: ops.linear(x, ws[i % copies], parts_ok=parts_ok)
        nbytes = n * k * 2
    else:
        hq, hkv, d, page = 32, 8, 128, PAGE
        if kind.startswith("attn_decode"):
            b, ctx = int(rest[0]), int(rest[1])
            split = int(rest[2]) if len(rest) > 2 else 256
            page = int(rest[3]) if len(rest) > 3 else PAGE
            if len(rest) > 4:
                hkv = int(rest[4]); hq = (int(rest[5]) if len(rest) > 5 else 4) * hkv
            q_lens = [1] * b
        else:
            b, ctx, q_lens = 1, 0, [int(rest[0])]
            page = int(rest[1]) if len(rest) > 1 else PAGE
        total = [ctx + q for q in q_lens]
        pages_per = [-(-t // page) for t in total]
        num_pages = sum(pages_per)
        table = torch.full((b, max(pages_per)), -1, dtype=torch.int32)
        perm = torch.randperm(num_pages).tolist()
        for e in range(b):
            for i in range(pages_per[e]):
                table[e, i] = perm.pop()
        copies = max(1, int(300e6 // (num_pages * page * hkv * d * 4))) + 1 if kind.startswith("attn_decode") else 1
        kcs = [torch.randn(num_pages, page, hkv, d, device=dev).to(torch.bfloat16) for _ in range(copies)]
        vcs = [torch.randn(num_pages, page, hkv, d, device=dev).to(torch.bfloat16) for _ in range(copies)]
        kc, vc = kcs[0], vcs[0]
        n_tok = sum(q_lens)
        q = torch.randn(n_tok, hq * d, device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=dev)
        st = torch.tensor([ctx] * b, dtype=torch.int32, device=dev)
        common = (kc, vc, table.to(dev), cu, st)
        if kind.startswith("attn_decode"):
            work = torch.tensor([[e, 0] for e in range(b)], dtype=torch.int32, device=dev)
            n_splits = -(-max(total) // split)
            if kind == "attn_decode_tcgen05":
                run = lambda i: ops.attn_decode_tcgen05(q, hq * d, out, kcs[i % copies], vcs[i % copies], *common[2:], work,
                                                        b, hq, hkv, d, d ** -0.5)
            else:
                run = lambda i: ops.attn_mma(q, hq * d, out, kcs[i % copies], vcs[i % copies], *common[2:], work, b, hq,
                                             hkv, d, 0, d ** -0.5, split_size=split, n_splits=n_splits)
        elif kind == "attn_prefill_tcgen05":
            tpt = ops.attn_tcgen05_tokens_per_tile(hq, hkv)
            work = torch.tensor([[0, t] for t in range(0, q_lens[0], tpt)], dtype=torch.int32, device=dev)
            run = lambda i: ops.attn_tcgen05(q, hq * d, out, *common, work, work.shape[0], hq, hkv, d, d ** -0.5)
        else:
            tpt = ops.attn_mma_tokens_per_tile(hq, hkv)
            work = torch.tensor([[0, t] for t in range(0, q_lens[0], tpt)], dtype=torch.int32, device=dev)
            run = lambda i: ops.attn_mma(q, hq * d, out, *common, work, work.shape[0], hq, hkv, d, 0, d ** -0.5)
        nbytes = 2 * kc.numel() * 2
    for i in range(3):
        run(i)
    torch.cuda.synchronize()
    if (kind.startswith("attn_decode") or kind == "linear") and not eager:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(copies):
                run(i)
        graph.replay()
        torch.cuda.synchronize()
        start.record()
        for i in range(reps):
            graph.replay()
        end.record()
        reps *= copies
    else:
        start.record()
        for i in range(reps):
            run(i)
        end.record()
    torch.cuda.synchronize()
    ops.check_status()
    us = start.elapsed_time(end) / reps * 1e3
    print(json.dumps({"micro": spec, "us": round(us, 2), "GB/s": round(nbytes / us / 1e3, 1)}))
    return 0


def timeline(batch: int, layers: int, shape=None) -> int:
    """Start, duration and end of every kernel of one replayed decode step (torch's profiler; programmatic dependent
    launch lets kernels overlap, so a kernel's start is when its first block became resident, and the increments from
    end to end tell what each adds to the step): `python bench.py --timeline 8 --layers 4`; with `--workload NAME`
    the layer sizes of that workload's shape instead of the 8B ones."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    from jax_vllm_b200 import make_driver, random_model, registry
    from jax_vllm_b200.engine import StepEntry
    cfg = dict(QWEN3_8B, **(WORKLOADS[shape]["config"] if shape else {}))
    model = random_model(registry.config_from_dict(dict(cfg, num_hidden_layers=layers)), seed=5, dtype="bf16")
    driver = make_driver(model, max_num_seqs=batch, max_model_len=CONTEXT + 64, block_size=PAGE, prefix_cache=False)
    rcs = fake_context(driver, batch, CONTEXT)

    def one(i):
        entries = []
        for b, rc in enumerate(rcs):
            driver.cache.grow(rc, rc.num_tokens + 1)
            entries.append(StepEntry(rc, [(i * 7919 + b) % 1000], (0,)))
        driver.runner.step(entries)
        for rc in rcs:
            rc.num_tokens += 1

    for i in range(6):
        one(i)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        one(7)
        torch.cuda.synchronize()
    evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda e: e.time_range.start)
    t0, last_end = evs[0].time_range.start, evs[0].time_range.start
    print(f"decode step, batch {batch}, {CONTEXT}-token context, {layers} layers: start, duration, end, end minus the latest end before (us)")
    for e in evs:
        start, dur = e.time_range.start - t0, e.time_range.end - e.time_range.start
        print(f"{start:9.1f} {dur:7.1f} {start + dur:9.1f} {e.time_range.end - last_end:+7.1f}  {e.name[:70]}")
        last_end = max(last_end, e.time_range.end)
    return 0


WORKLOADS = {
    # the larger dense Qwen3 shapes as serving workloads: all requests arrive at once, the scheduler cuts their
    # prompts into portions beside the decode tokens of the others
    "mixed14b": dict(config=dict(hidden_size=5120, intermediate_size=17408, num_hidden_layers=40, num_attention_heads=40),
                     seed=6, requests=32, prompt=(128, 4096), prompt_seed=7, shared_prefix=1024, new_tokens=256,
                     tokens_per_step=512),
    "long32b": dict(config=dict(hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64),
                    seed=8, requests=16, prompt=(8192, 8192), prompt_seed=9, shared_prefix=0, new_tokens=512,
                    tokens_per_step=2048),
}


def workload(name: str, layers) -> int:
    """Runs one of WORKLOADS through the entry point and prints one JSON line: wall-clock seconds, prompt and
    generated tokens per second, time to the first token, and the steps by kind (with a portion of a prompt
    in them, or decoding alone) with their time and the tokens they ran."""
    import random
    import torch
    from jax_vllm_b200 import SamplingParams, add_request, has_work, make_driver, prewarm, random_model, registry, step
    w = WORKLOADS[name]
    cfg_dict = dict(QWEN3_8B, **w["config"])
    if layers:
        cfg_dict["num_hidden_layers"] = layers
    model = random_model(registry.config_from_dict(cfg_dict), seed=w["seed"], dtype="bf16", device="cuda:0")
    rng = random.Random(w["prompt_seed"])
    vocab = cfg_dict["vocab_size"]
    shared = [rng.randrange(vocab) for _ in range(w["shared_prefix"])]
    prompts = []
    for i in range(w["requests"]):
        n = rng.randint(*w["prompt"])
        own = [rng.randrange(vocab) for _ in range(n)]
        prompts.append((shared + own[len(shared):]) if shared and i % 2 == 0 and n > len(shared) else own)
    longest = max(len(p) for p in prompts)
    max_len = -(-(longest + w["new_tokens"]) // PAGE) * PAGE
    driver = make_driver(model, max_num_seqs=w["requests"], max_model_len=max_len, max_prefill_len=longest,
                         block_size=PAGE, max_tokens_per_step=w["tokens_per_step"])
    warm = prewarm(driver)
    torch.cuda.synchronize()
    st = driver.stats
    kinds = {"with_prompt": [0, 0.0, 0], "decode_only": [0, 0.0, 0]}          # steps, seconds, tokens run
    with ClockSampler() as clocks:
        t0 = time.perf_counter()
        ids = [add_request(driver, p, SamplingParams(max_new_tokens=w["new_tokens"])) for p in prompts]
        reqs = [driver.requests[i] for i in ids]
        while has_work(driver):
            t1 = time.perf_counter()
            before = (st.prefill_tokens, st.decode_tokens)
            step(driver)
            rec = kinds["with_prompt" if st.prefill_tokens > before[0] else "decode_only"]
            rec[0] += 1
            rec[1] += time.perf_counter() - t1
            rec[2] += st.prefill_tokens + st.decode_tokens - sum(before)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    n_prompt, n_new = sum(len(p) for p in prompts), sum(len(r.output_ids) for r in reqs)
    ttft = sorted(r.first_token_time - r.arrival for r in reqs)
    out = {"workload": name, "layers": cfg_dict["num_hidden_layers"], "requests": len(prompts), "prompt_tokens": n_prompt,
           "new_tokens": n_new, "seconds": round(dt, 3), "tokens_per_s": round((n_prompt + n_new) / dt, 1),
           "new_tokens_per_s": round(n_new / dt, 1),
           "ttft_s": {"median": round(ttft[len(ttft) // 2], 3), "max": round(ttft[-1], 3)}, "steps": st.steps}
    for kind, (n, sec, toks) in kinds.items():
        out["steps_" + kind] = {"steps": n, "ms_per_step": round(1e3 * sec / max(1, n), 2),
                                "tokens_per_s": round(toks / max(1e-9, sec), 1)}
    out.update({"preemptions": st.preemptions, "prefix_hit_tokens": st.cache_hit_tokens, "prewarm_s": round(warm, 1),
                "gb_allocated": round(torch.cuda.max_memory_allocated() / 1e9, 1),
                "clocks": clocks.summary})
    print(json.dumps(out))
    return 0


def reference_arm():
    why = ("the reference (jllm) needs jax, jaxlib and equinox and the hatchling build backend; none is installed "
           "and none is in the offline wheelhouse, so it can neither be installed nor run here")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the configuration has (same layer sizes), for a quick run")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64, and the prefill")
    ap.add_argument("--only-prefill", action="store_true", help="time the 2,048-token prefill alone (for profiling)")
    ap.add_argument("--micro", default=None, help="run one kernel alone, e.g. linear:24576x4096:8 (see micro())")
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="a serving workload of a larger shape through the entry point (see WORKLOADS); --layers cuts it")
    ap.add_argument("--timeline", type=int, default=None, metavar="BATCH",
                    help="print every kernel of one replayed decode step at this batch with its start and end (use --layers)")
    ap.add_argument("--with-workloads", action="store_true",
                    help="after the headline run, also run the two serving workloads and add their lines under `workloads`")
    ap.add_argument("--micro-eager", action="store_true",
                    help="with --micro: plain launches instead of replays of a CUDA graph (for a profiler)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.micro:
        return micro(args.micro, max(1, args.steps), args.micro_eager)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.timeline:
        return timeline(args.timeline, args.layers or 4, args.workload)
    if args.workload:
        return workload(args.workload, args.layers)
    args.layers = args.layers or QWEN3_8B["num_hidden_layers"]
    warmup = max(3, args.warmup)

    import torch
    from jax_vllm_b200 import random_model, registry

    cfg_dict = dict(QWEN3_8B, num_hidden_layers=args.layers)
    cfg = registry.config_from_dict(cfg_dict)
    model = random_model(cfg, seed=5, dtype="bf16", device="cuda:0")
    pk, pk_src = peaks()
    if args.only_prefill:
        pms = time_prefill(model, PREFILL_TOKENS, warmup=1, reps=max(1, args.steps))
        print(json.dumps({"prefill_ms": round(pms, 3), "tokens": PREFILL_TOKENS, "layers": args.layers}))
        return 0

    region_clocks = {}
    with ClockSampler() as clocks:
        ms, launches, repeats, all_ms = time_decode(model, args.batch, args.steps, warmup)
    region_clocks["decode"] = clocks.summary
    value = args.batch / (ms / 1e3)
    bytes_step = decode_bytes(cfg_dict, args.layers, args.batch, CONTEXT + warmup + repeats * args.steps // 2)
    achieved = bytes_step / (ms / 1e3) / 1e9
    out = {
        "metric": f"decode tok/s (Qwen3-8B shape, bf16, batch {args.batch}, {CONTEXT}-token context)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "repeats": repeats, "ms_per_step_of_repeats": [round(v, 4) for v in all_ms],
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (uniform random token ids, random N(0,0.02) weights, seed 5)",
        "config": {"model": "Qwen3-8B shape", "layers": args.layers, "layers_of_config": QWEN3_8B["num_hidden_layers"],
                   "hidden": 4096, "q_heads": 32, "kv_heads": 8, "head_dim": 128, "intermediate": 12288,
                   "vocab": 151936, "global_batch": args.batch, "seq_len": CONTEXT, "max_context": 4096,
                   "page_size": PAGE, "parallelism": "none (1 GPU)", "l2": "inputs larger than L2 (15 GB of weights)",
                   "cuda_graphs": True, "timed": f"median of {repeats} repeats of {args.steps} steps"},
        "gpu_launches": launches * args.steps * repeats,
        "clocks": clocks.summary,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk_src},
    }
    if not args.skip_points:
        with ClockSampler() as c:
            e2e, e2e_best, runs, h2d, d2h = time_e2e(model, args.batch, args.steps, warmup)
        region_clocks["e2e"] = c.summary
        out["e2e"] = {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                      "runs": runs, "picked": "median over the runs of `steps` steps", "best": round(e2e_best, 1)}
        with ClockSampler() as c:
            pms = time_prefill(model, PREFILL_TOKENS, warmup=2, reps=max(3, int(MIN_TIMED_SECONDS / 0.027)))
        region_clocks["prefill"] = c.summary
        flops = prefill_flops(cfg_dict, args.layers, PREFILL_TOKENS)
        out["prefill"] = {"value": round(PREFILL_TOKENS / (pms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pms, 3),
                          "frac": round(flops / (pms / 1e3) / 1e12 / pk["bf16_tflops"], 4),
                          "peak_tflops": pk["bf16_tflops"], "peak_source": pk_src}
        points = {}
        for b in (1, 64):
            with ClockSampler() as c:
                pms_b, _, _, _ = time_decode(model, b, max(8, args.steps // 2), warmup)
            region_clocks[f"decode_b{b}"] = c.summary
            points[f"decode_b{b}"] = round(b / (pms_b / 1e3), 1)
            frac = decode_bytes(cfg_dict, args.layers, b, CONTEXT + 64) / (pms_b / 1e3) / 1e9 / pk["hbm_gbs"]
            points[f"decode_b{b}_hbm_frac"] = round(frac, 4)
        out["points"] = points
    out["clocks_by_region"] = region_clocks
    if args.with_workloads:
        # the two serving workloads of larger shapes, each in a process of its own (they need the device's memory)
        del model
        torch.cuda.empty_cache()
        out["workloads"] = {}
        for name in sorted(WORKLOADS):
            proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--workload", name], capture_output=True, text=True)
            line = [l for l in proc.stdout.splitlines() if l.startswith("{")]
            out["workloads"][name] = json.loads(line[-1]) if proc.returncode == 0 and line else {"failed": proc.stderr[-300:]}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
