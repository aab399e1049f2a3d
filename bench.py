"""Decode and prefill throughput of the engine on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step: every live request gets one token.  The default run
has the layer sizes of Qwen3-8B (36 layers, hidden 4096, 32/8 heads of 128,
intermediate 12288, vocabulary 151936, untied head) with random bfloat16 weights,
8 requests at a context of 8192 tokens, pages of 16.  One JSON line is printed:
``value`` is decoded tokens per second timed on the device over K graph-replayed
steps; ``e2e`` is the same through ``Engine.step`` with host token ids in and
sampled ids out; ``prefill`` times one 2048-token prompt; ``roofline`` relates the
bytes a decode step must read (every weight once, the cache of the live requests)
to the measured copy bandwidth; ``points`` holds decode at batch 1 and 64 at the same
context and at batch 16, 32 and 64 at a context of 1024 (tokens per second), and
``points_detail`` their milliseconds, bytes and fraction of the copy bandwidth.
Peaks come from MEASURED_PEAKS.json beside this file when present.
``--shape 32b|0.6b`` prints the same line for the other layer sizes; ``--impl reference``
the same line for the unmodified reference engine.
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

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}

QWEN3_8B = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=40960,
                rms_norm_eps=1e-6, rope_theta=1000000.0, attention_bias=False, tie_word_embeddings=False,
                eos_token_id=None)
QWEN3_32B = dict(QWEN3_8B, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64)
QWEN3_06B = dict(QWEN3_8B, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
                 tie_word_embeddings=True)
# name -> (sizes, label, context of the decode measurements)
SHAPES = {"8b": (QWEN3_8B, "Qwen3-8B shape", 8192), "32b": (QWEN3_32B, "Qwen3-32B shape", 8192),
          "0.6b": (QWEN3_06B, "Qwen3-0.6B shape", 4096)}
CONTEXT = 8192
PAGE_SIZE = 16
PREFILL_TOKENS = 2048


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            flat = {}
            def walk(node):
                if isinstance(node, dict):
                    for key, value in node.items():
                        if isinstance(value, (int, float)) and key not in flat:
                            flat[key] = float(value)
                        else:
                            walk(value)
                elif isinstance(node, list):
                    for item in node:
                        walk(item)
            walk(data)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return {"hbm_gbs": flat["hbm_gbs"], "bf16_tflops": flat["bf16_tflops"],
                        "bf16_tflops_sustained": flat.get("bf16_tflops_sustained"), "source": "measured"}
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines, self.proc, self.thread = [], None, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0],
                                          f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        mhz, max_mhz, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6 or not parts[0].isdigit():
                continue
            mhz.append(int(parts[0])); max_mhz.append(int(parts[1]))
            for name, value in zip(names, parts[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        if not mhz:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": int(statistics.median(mhz)), "sm_max_mhz": max(max_mhz), "reasons": sorted(reasons)}


def gemm_params(cfg):
    """Matrix elements every token passes through: the four projections of each layer and the head."""
    h, d = cfg["hidden_size"], cfg["head_dim"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * d * h
    o = cfg["num_attention_heads"] * d * h
    mlp = 3 * cfg["intermediate_size"] * h
    return cfg["num_hidden_layers"] * (qkv + o + mlp), cfg["vocab_size"] * h


def decode_bytes(cfg, batch, context, dtype_bytes=2):
    layer_params, head_params = gemm_params(cfg)
    norms = cfg["num_hidden_layers"] * (2 * cfg["hidden_size"] + 2 * cfg["head_dim"]) + cfg["hidden_size"]
    kv_per_token = cfg["num_hidden_layers"] * 2 * cfg["num_key_value_heads"] * cfg["head_dim"]
    return dtype_bytes * (layer_params + head_params + norms + batch * context * kv_per_token)


def prefill_flops(cfg, tokens, logit_rows=1):
    layer_params, head_params = gemm_params(cfg)
    gemm = 2.0 * tokens * layer_params + 2.0 * logit_rows * head_params
    attention = cfg["num_hidden_layers"] * 4.0 * cfg["num_attention_heads"] * cfg["head_dim"] * tokens * (tokens + 1) / 2
    return gemm + attention


def config_record(cfg, label, batch, context, full_layers, of):
    """The ``config`` of a bench line: every size by name, flat; the same keys for both arms."""
    return {"model": label, "layers": cfg["num_hidden_layers"], "layers_of_config": full_layers,
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "tied": cfg["tie_word_embeddings"],
            "global_batch": batch, "seq_len": context, "page_size": PAGE_SIZE, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (decode reads >16 GB per step); prefill flushes a 256 MB buffer",
            "peaks": of}


# --------------------------------------------------------------------------- our engine
class OursBench:
    def __init__(self, cfg, layers=None, dtype="bfloat16"):
        import torch
        from qwen_inference_lab_b200.config import Qwen3Config
        from qwen_inference_lab_b200.loading import random_model
        self.torch = torch
        self.cfg = dict(cfg)
        self.full_layers = cfg["num_hidden_layers"]
        if layers:
            self.cfg["num_hidden_layers"] = layers
        self.dtype = getattr(torch, dtype)
        self.model = random_model(Qwen3Config.from_dict(dict(self.cfg, model_type="qwen3")), seed=0,
                                  device="cuda", dtype=self.dtype)
        torch.cuda.synchronize()

    def largest_context(self, batch, wanted, reserve=6 << 30):
        """The longest context (a multiple of 1024, at most ``wanted``) whose cache for ``batch`` requests fits."""
        free, _ = self.torch.cuda.mem_get_info()
        per_token = (self.cfg["num_hidden_layers"] * 2 * self.cfg["num_key_value_heads"] * self.cfg["head_dim"]
                     * self.dtype.itemsize)
        fits = int((free - reserve) // (batch * per_token)) // 1024 * 1024
        return max(1024, min(wanted, fits))

    def _fill_cache(self, cache, ids, context):
        for g in cache.kv_groups:
            g.storage.normal_(0.0, 0.5)
        for rid in ids:
            assert cache.admit(rid)
            cache.ensure(rid, context)
            cache.advance(rid, context)

    def decode(self, batch, context, steps, warmup, sample_clocks=False):
        """Device-timed decode: K steps of ``batch`` single tokens at ``context`` cached tokens each."""
        torch = self.torch
        from qwen_inference_lab_b200.cache import CacheManager
        from qwen_inference_lab_b200.engine import StepEntry, StepRunner
        from qwen_inference_lab_b200.kernels import ops
        total = context + steps + warmup + 2
        pages_per_request = (total + PAGE_SIZE - 1) // PAGE_SIZE
        cache = CacheManager(self.model.cache_specs(), num_pages=batch * pages_per_request, page_size=PAGE_SIZE,
                             max_requests=batch, max_context=pages_per_request * PAGE_SIZE, dtype=self.dtype,
                             device=self.model.device)
        runner = StepRunner(self.model, cache, max_step_tokens=max(batch, 64))
        ids = list(range(batch))
        self._fill_cache(cache, ids, context)
        generator = torch.Generator().manual_seed(1)
        tokens = torch.randint(0, self.cfg["vocab_size"], (steps + warmup + 1, batch), generator=generator).tolist()
        def one(i):
            return runner.run([StepEntry(rid, [tokens[i][rid]], [0]) for rid in ids])
        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        launches_before = ops.launch_count()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler = ClockSampler() if sample_clocks else None
        if sampler:
            sampler.__enter__()
        torch.cuda.synchronize()
        start.record()
        for i in range(warmup, warmup + steps):
            logits = one(i)
        stop.record()
        torch.cuda.synchronize()
        if sampler:
            sampler.__exit__()
        ms = start.elapsed_time(stop) / steps
        assert torch.isfinite(logits).all()
        per_step = getattr(runner, "launches_per_graph", {}).get(batch)
        result = dict(ms_per_step=ms, tokens_per_s=batch / ms * 1e3,
                      bytes=decode_bytes(self.cfg, batch, context + warmup + steps // 2, self.dtype.itemsize),
                      launches=per_step * steps if per_step else ops.launch_count() - launches_before,
                      clocks=sampler.summary() if sampler else None)
        del runner, cache
        torch.cuda.empty_cache()
        return result

    def prefill(self, tokens_n, reps=9, warmup=4):
        torch = self.torch
        from qwen_inference_lab_b200.cache import CacheManager
        from qwen_inference_lab_b200.engine import StepEntry, StepRunner
        pages = (tokens_n + PAGE_SIZE - 1) // PAGE_SIZE + 1
        cache = CacheManager(self.model.cache_specs(), num_pages=pages, page_size=PAGE_SIZE, max_requests=2,
                             max_context=pages * PAGE_SIZE, dtype=self.dtype, device=self.model.device)
        runner = StepRunner(self.model, cache, max_step_tokens=tokens_n)
        generator = torch.Generator().manual_seed(2)
        prompt = torch.randint(0, self.cfg["vocab_size"], (tokens_n,), generator=generator).tolist()
        times = []
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        sampler = ClockSampler()
        sampler.__enter__()
        for i in range(warmup + reps):
            cache.admit("p")
            flush.zero_()   # a buffer larger than L2 between timed iterations
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            logits = runner.run([StepEntry("p", prompt, [tokens_n - 1])])
            stop.record()
            torch.cuda.synchronize()
            cache.release("p")
            if i >= warmup:
                times.append(start.elapsed_time(stop))
        sampler.__exit__()
        self.last_prefill_clocks = sampler.summary()
        assert torch.isfinite(logits).all()
        ms = statistics.median(times)
        self.last_prefill_times = sorted(round(t, 3) for t in times)
        del runner, cache, flush
        torch.cuda.empty_cache()
        return ms

    def e2e(self, batch, context, steps, warmup):
        """Decode through Engine.step: host token ids in (pinned staging), sampled ids out, every step."""
        torch = self.torch
        from qwen_inference_lab_b200 import Engine
        new_tokens = steps + warmup + 4
        prompt_len = context - 1
        pages = batch * ((prompt_len + new_tokens + PAGE_SIZE - 1) // PAGE_SIZE + 1)
        engine = Engine(self.model, num_pages=pages, page_size=PAGE_SIZE, token_budget=2048, prefill_chunk=2048,
                        max_active=batch, overlap=True)       # a step ahead of the host, as generate() runs
        generator = torch.Generator().manual_seed(3)
        for _ in range(batch):
            prompt = torch.randint(0, self.cfg["vocab_size"], (prompt_len,), generator=generator).tolist()
            engine.submit(prompt, max_new_tokens=new_tokens, ignore_eos=True)
        while engine.scheduler.prefilling:
            engine.step()
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        begin = time.perf_counter()
        emitted = 0
        for _ in range(steps):
            emitted += len(engine.step())
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - begin
        h2d = engine.runner.last_upload_bytes
        engine.close()
        del engine
        torch.cuda.empty_cache()
        return dict(value=emitted / elapsed, unit="tokens/s", h2d_bytes_per_step=h2d, d2h_bytes_per_step=2 * 4 * batch,
                    ms_per_step=elapsed / steps * 1e3)


def mixed_workload(bench, requests=64, new_tokens=128, longest=2048, seed=4):
    """Requests with prompts of 16 to ``longest`` tokens (uniform, seeded), ``new_tokens`` each, all
    submitted at once to ``Engine.generate``: output tokens per second of the whole run, wall clock."""
    import torch
    from qwen_inference_lab_b200 import Engine
    generator = torch.Generator().manual_seed(seed)
    lengths = torch.randint(16, longest + 1, (requests,), generator=generator).tolist()
    prompts = [torch.randint(0, bench.cfg["vocab_size"], (n,), generator=generator).tolist() for n in lengths]
    pages = sum((n + new_tokens + PAGE_SIZE - 1) // PAGE_SIZE + 1 for n in lengths)
    engine = Engine(bench.model, num_pages=pages, page_size=PAGE_SIZE, token_budget=4096, prefill_chunk=2048,
                    max_active=requests)
    # set-up outside the timed run, as the reference's harness keeps load and warm-up out of its samples
    # (docs/batched-gpu-validation-2026-09-20.md:19-24): the same workload once, which also records the decode
    # steps' graphs for the batch sizes and context ranges it passes through
    engine.generate(prompts, max_new_tokens=new_tokens, ignore_eos=True)
    torch.cuda.synchronize()
    steps_before = engine.runner.steps_run
    begin = time.perf_counter()
    rows = engine.generate(prompts, max_new_tokens=new_tokens, ignore_eos=True)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - begin
    produced = sum(len(row["token_ids"]) for row in rows)
    steps = engine.runner.steps_run - steps_before
    engine.close()
    return {"value": round(produced / elapsed, 1), "unit": "output tokens/s", "requests": requests,
            "prompt_tokens": sum(lengths), "new_tokens": produced, "steps": steps, "seconds": round(elapsed, 3)}


def run_ours(args):
    import torch
    pk = peaks()
    sizes, label, context = SHAPES[args.shape]
    bench = OursBench(sizes, layers=args.layers, dtype=args.dtype)
    cfg = bench.cfg
    batch = args.batch
    if args.only == "mixed":
        print(json.dumps({"workload": "mixed", "model": label, "dtype": args.dtype, **mixed_workload(bench)}))
        return
    if args.only == "decode":
        part = bench.decode(batch, args.context, args.steps, args.warmup)
        print(f"decode batch {batch} context {args.context} layers {cfg['num_hidden_layers']}: {part['ms_per_step']:.3f} ms/step")
        return
    if args.only == "prefill":
        ms = bench.prefill(args.prefill_tokens, reps=args.steps if args.steps != 32 else 2, warmup=3)
        frac = prefill_flops(cfg, args.prefill_tokens) / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12)
        print(f"prefill {args.prefill_tokens} tokens layers {cfg['num_hidden_layers']}: {ms:.3f} ms "
              f"({args.prefill_tokens / ms * 1e3:.0f} tokens/s, {frac:.3f} of the bf16 peak; all: {bench.last_prefill_times})")
        return
    main = bench.decode(batch, context, args.steps, args.warmup, sample_clocks=True)
    points, points_detail = {}, {}
    short = min(1024, context)
    for b, wanted in ((1, context), (64, context), (16, short), (32, short), (64, short)):
        if args.quick:
            break
        fits = bench.largest_context(b, wanted)      # the 32B shape holds 64 requests only at a shorter context
        key = f"decode_b{b}" if fits == context else f"decode_b{b}_context{fits}"
        part = bench.decode(b, fits, max(8, args.steps // 2), args.warmup)
        points[key] = round(part["tokens_per_s"], 1)
        gbs = part["bytes"] / (part["ms_per_step"] * 1e-3) / 1e9
        points_detail[key] = {"ms": round(part["ms_per_step"], 4), "gbytes": round(part["bytes"] / 1e9, 3),
                              "gbs": round(gbs, 1), "frac": round(gbs / pk["hbm_gbs"], 4)}
    prefill_ms = bench.prefill(PREFILL_TOKENS)
    e2e = bench.e2e(batch, context, args.steps, args.warmup)
    flops = prefill_flops(cfg, PREFILL_TOKENS)
    achieved = main["bytes"] / (main["ms_per_step"] * 1e-3) / 1e9
    of = "of measured" if pk["source"] == "measured" else "of fallback"
    line = {
        "metric": f"decode tokens/s ({label}, batch {batch}, context {context})",
        "value": round(main["tokens_per_s"], 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic: random weights, random token ids, random cache contents",
        "impl": "ours",
        "config": config_record(cfg, label, batch, context, bench.full_layers, of),
        "clocks": main["clocks"],
        "e2e": {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": int(main["launches"]),
        "prefill": {"value": round(PREFILL_TOKENS / prefill_ms * 1e3, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3),
                    # the peak is the bfloat16 tensor-core one: no fraction for the float32 check path
                    "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4) if args.dtype == "bfloat16" else None,
                    "ms_min": bench.last_prefill_times[0], "ms_max": bench.last_prefill_times[-1],
                    "sm_mhz": bench.last_prefill_clocks["sm_mhz"], "reasons": bench.last_prefill_clocks["reasons"]},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "points_detail": points_detail,
    }
    print(json.dumps(line), flush=True)



# --------------------------------------------------------------------------- Virulix beside dense Qwen3
def _virulix_sizes(width, heads, kv_heads, dim, gla_heads, gla_vdim, dense_ff, experts, top, expert_ff, shared_ff, vocab):
    """Eight layers that use every mechanism of the design at one width."""
    attention = lambda **extra: dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=dim ** -0.5,
                                     q_temp=dict(coef=0.1, every=256), **extra)
    gla = dict(heads=gla_heads, dim=dim, vdim=gla_vdim, tau=16.0, rank=16)
    moe = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=expert_ff, limit=7.0),
               shared=dict(ff=shared_ff, limit=7.0))
    dense = dict(kind="dense", ff=dense_ff)
    layers = [dict(type="attention", mixer=attention(), mlp=dense), dict(type="gla", mixer=gla, mlp=moe),
              dict(type="attention", mixer=attention(), mlp=moe), dict(type="gla", mixer=gla, mlp=moe),
              dict(type="attention", mixer=attention(kv_from=2), mlp=moe), dict(type="gla", mixer=gla, mlp=dense),
              dict(type="attention", mixer=attention(), mlp=dense), dict(type="gla", mixer=gla, mlp=moe)]
    return dict(architecture="Virulix", vocab=vocab, width=width, norm=dict(eps=1e-6), layers=layers)


VIRULIX_SHAPES = {
    # name: (Virulix sizes, the dense Qwen3 of equal width, heads, head size, layer count and vocabulary)
    "2048": dict(width=2048, heads=16, kv_heads=4, dim=128, gla_heads=4, gla_vdim=256, dense_ff=6144, experts=32,
                 top=4, expert_ff=768, shared_ff=1536, vocab=32768),
    "4096": dict(width=4096, heads=32, kv_heads=8, dim=128, gla_heads=8, gla_vdim=256, dense_ff=12288, experts=64,
                 top=6, expert_ff=1024, shared_ff=2048, vocab=32768),
}


def _timed(torch, fn, reps=12, warmup=3, flush=None):
    """Median milliseconds of ``fn`` on the device, an L2 flush before every timed call."""
    times = []
    for i in range(warmup + reps):
        if flush is not None:
            flush.zero_()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(start.elapsed_time(stop))
    return statistics.median(times)


class _ModelBench:
    """Whole-model prompt and decode steps of any model of the engine, timed on the device."""

    def __init__(self, model, vocab):
        import torch
        self.torch, self.model, self.vocab = torch, model, vocab

    def _parts(self, tokens, requests):
        from qwen_inference_lab_b200.cache import CacheManager
        from qwen_inference_lab_b200.engine import StepRunner
        pages = requests * ((tokens + PAGE_SIZE - 1) // PAGE_SIZE + 2)
        cache = CacheManager(self.model.cache_specs(), num_pages=pages, page_size=PAGE_SIZE, max_requests=requests,
                             max_context=pages * PAGE_SIZE, dtype=self.model.dtype, device=self.model.device)
        return cache, StepRunner(self.model, cache, max_step_tokens=max(tokens, 64))

    def prefill(self, tokens_n, flush):
        from qwen_inference_lab_b200.engine import StepEntry
        torch = self.torch
        cache, runner = self._parts(tokens_n, 1)
        prompt = torch.randint(0, self.vocab, (tokens_n,), generator=torch.Generator().manual_seed(2)).tolist()
        def once():
            cache.admit("p")
            runner.run([StepEntry("p", prompt, [tokens_n - 1])])
            cache.release("p")
        return _timed(torch, once, reps=7, warmup=3, flush=flush)

    def decode(self, batch, context, steps, warmup):
        from qwen_inference_lab_b200.engine import StepEntry
        torch = self.torch
        cache, runner = self._parts(context + steps + warmup + 2, batch)
        for g in cache.kv_groups:
            g.storage.normal_(0.0, 0.5)
        for rid in range(batch):
            cache.admit(rid)
            cache.ensure(rid, context)
            cache.advance(rid, context)
        tokens = torch.randint(0, self.vocab, (steps + warmup, batch), generator=torch.Generator().manual_seed(1)).tolist()
        one = lambda i: runner.run([StepEntry(rid, [tokens[i][rid]], [0]) for rid in range(batch)])
        for i in range(warmup):
            one(i)
        # every step between its own pair of events, the median of them: a step that waits for the allocator
        # (a new graph pool, a library's workspace) does not count for sixteen
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        torch.cuda.synchronize()
        marks[0].record()
        for i in range(warmup, warmup + steps):
            logits = one(i)
            marks[i - warmup + 1].record()
        torch.cuda.synchronize()
        assert torch.isfinite(logits).all()
        return statistics.median(a.elapsed_time(b) for a, b in zip(marks, marks[1:]))


def _mixer_kernels(torch, model, sizes, pk, tokens_n, batch, context, flush, qwen):
    """The mixers' own kernels alone, with what the roofline allows: (name, ms, fraction of the measured peak)."""
    from qwen_inference_lab_b200.cache import CacheManager
    from qwen_inference_lab_b200.engine import StepEntry, StepRunner
    from qwen_inference_lab_b200.kernels import ops
    from tests.harness import OnePartModel
    rows = []
    H, G, d = sizes["heads"], sizes["kv_heads"], sizes["dim"]
    tflops, gbs = pk["bf16_tflops"] * 1e12, pk["hbm_gbs"] * 1e9

    def run_part(part, body, hidden, prompt_tokens, decode_batch, decode_context):
        """(ms of a whole prompt, ms of a step of single tokens) of ``body`` over the step function."""
        shell = OnePartModel(part, hidden, torch.bfloat16, body)
        shell.inputs = torch.randn(4096, hidden, device="cuda").to(torch.bfloat16)
        pages = (decode_batch + 1) * ((max(prompt_tokens, decode_context) + PAGE_SIZE) // PAGE_SIZE + 2)
        cache = CacheManager(shell.cache_specs(), num_pages=pages, page_size=PAGE_SIZE, max_requests=decode_batch + 1,
                             max_context=pages * PAGE_SIZE, dtype=torch.bfloat16, device="cuda")
        for g in cache.kv_groups:
            g.storage.normal_(0.0, 0.5)
        runner = StepRunner(shell, cache, max_step_tokens=prompt_tokens, use_graphs=False)
        ids = [i % 4096 for i in range(prompt_tokens)]
        def prompt():
            cache.admit("p")
            runner.run([StepEntry("p", ids, [])])
            cache.release("p")
        for rid in range(decode_batch):
            cache.admit(rid)
            cache.ensure(rid, decode_context)
            cache.advance(rid, decode_context)
        single = lambda: runner.run([StepEntry(rid, [rid], []) for rid in range(decode_batch)])
        return prompt, single, shell

    class Timer:
        """Times the part's kernel inside ``body`` with events of its own, so that the projections around it stay out."""
        def __init__(self):
            self.ms = []
        def __call__(self, fn):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            out = fn()
            stop.record()
            self.ms.append((start, stop))
            return out
        def median(self, skip):
            torch.cuda.synchronize()
            values = [a.elapsed_time(b) for a, b in self.ms[skip:]]
            self.ms = []
            return statistics.median(values)

    def measure(name_prefix, part, hidden, kernel_of, flops_prompt, bytes_decode):
        timer = Timer()
        def body(ctx, x, view):
            return kernel_of(ctx, x, view, timer)
        prompt, single, shell = run_part(part, body, hidden, tokens_n, batch, context)
        for i in range(8):
            flush.zero_()
            prompt()
            shell.outputs.clear()
        ms = timer.median(3)
        rows.append((f"{name_prefix} prompt {tokens_n}", ms, flops_prompt / (ms * 1e-3) / tflops, "of the bf16 peak"))
        for i in range(12):
            flush.zero_()
            single()
            shell.outputs.clear()
        ms = timer.median(4)
        rows.append((f"{name_prefix} decode b{batch} c{context}", ms, bytes_decode / (ms * 1e-3) / gbs, "of the copy bandwidth"))

    def attention_kernel(mixer):
        def kernel(ctx, x, view, timer):
            q = x[:, :H * d].contiguous()
            out = torch.empty_like(q)
            timer(lambda: mixer._attend(ctx, q, view, out))
            return out
        return kernel

    layers = model.layers
    attention = next(l.mixer for l in layers if hasattr(l.mixer, "plain_tail") and not l.mixer.reads_shared_cache)
    attn_flops = 4.0 * H * d * tokens_n * (tokens_n + 1) / 2
    attn_bytes = batch * context * 2 * G * d * 2
    measure("virulix attention (distance bias)", attention, H * d, attention_kernel(attention), attn_flops, attn_bytes)
    measure("qwen3 attention", qwen.layers[0].mixer, H * d, attention_kernel(qwen.layers[0].mixer), attn_flops, attn_bytes)

    gla = next(l.mixer for l in layers if hasattr(l.mixer, "decay_rank"))
    gh, gd, ge = gla.n_heads, gla.key_dim, gla.value_dim
    width = gla.projection.out_features
    def gla_kernel(ctx, x, view, timer):
        projected = x[:, :width].contiguous()
        mixed = torch.empty((x.shape[0], gh * ge), dtype=x.dtype, device=x.device)
        timer(lambda: gla.scan(ctx, projected, view, mixed))
        return mixed
    # the recurrence is float32 on the CUDA cores by the design: its prompt bound is the float32 FMA rate
    fma_peak = 148 * 128 * 2 * 1.9e9
    timer_rows = len(rows)
    measure("virulix gla scan", gla, max(width, 8), gla_kernel, 5.0 * gh * gd * ge * tokens_n, batch * gh * gd * ge * 4 * 2)
    name, ms, _, _ = rows[timer_rows]
    rows[timer_rows] = (name, ms, 5.0 * gh * gd * ge * tokens_n / (ms * 1e-3) / fma_peak, "of the float32 FMA rate (72 TFLOP/s nominal)")

    moe = next(l.feed_forward for l in layers if hasattr(l.feed_forward, "n_experts"))
    W, ff, E, top = moe.hidden_size, moe.expert_size, moe.n_experts, moe.top
    def moe_kernel(ctx, x, view, timer):
        h = x[:, :W].contiguous()
        chosen, weights = ops.moe_route(h, moe.router.data, moe.router_bias.data, top)
        return timer(lambda: ops.moe_experts(h, chosen, weights, moe._gate, moe._up, moe._down, moe.activation,
                                             limit=moe.limit, alpha=moe.alpha))
    measure("virulix routed experts", moe, W, moe_kernel, 2.0 * tokens_n * top * 3 * ff * W,
            min(E, batch * top) * 3 * ff * W * 2)
    dense = qwen.layers[0].feed_forward
    def dense_kernel(ctx, x, view, timer):
        h = x[:, :W].contiguous()
        return timer(lambda: dense.forward(ctx, h))
    inner = dense.intermediate_size
    measure("qwen3 gated mlp", dense, W, dense_kernel, 2.0 * tokens_n * 3 * inner * W, 3 * inner * W * 2)
    return rows


def run_virulix(args):
    """Prefill and decode of Virulix at sizes like a real model's layers, beside dense Qwen3 of equal width,
    heads, layer count and vocabulary, and the mixers' own kernels against their rooflines."""
    import torch
    from qwen_inference_lab_b200.config import Qwen3Config, VirulixConfig
    from qwen_inference_lab_b200.loading import random_model
    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for name in ([args.virulix_shape] if args.virulix_shape else sorted(VIRULIX_SHAPES)):
        sizes = VIRULIX_SHAPES[name]
        virulix = random_model(VirulixConfig.from_dict(_virulix_sizes(**sizes)), seed=0, device="cuda", dtype=torch.bfloat16)
        qwen_cfg = dict(QWEN3_8B, vocab_size=sizes["vocab"], hidden_size=sizes["width"], intermediate_size=sizes["dense_ff"],
                        num_hidden_layers=8, num_attention_heads=sizes["heads"], num_key_value_heads=sizes["kv_heads"],
                        head_dim=sizes["dim"])
        qwen = random_model(Qwen3Config.from_dict(dict(qwen_cfg, model_type="qwen3")), seed=0, device="cuda", dtype=torch.bfloat16)
        result = {"workload": "virulix", "width": sizes["width"], "layers": 8, "dtype": "bfloat16",
                  "peaks": "of measured" if pk["source"] == "measured" else "of fallback", "models": {}, "kernels": []}
        for label, model in (("virulix", virulix), ("qwen3", qwen)):
            bench = _ModelBench(model, sizes["vocab"])
            entry = {}
            for tokens_n in (512, 2048):
                ms = bench.prefill(tokens_n, flush)
                entry[f"prefill_{tokens_n}"] = {"ms": round(ms, 3), "tokens_per_s": round(tokens_n / ms * 1e3, 1)}
            for batch, context in ((1, 2048), (8, 2048), (32, 2048)):
                ms = bench.decode(batch, context, args.steps, max(args.warmup, 6))
                entry[f"decode_b{batch}_c{context}"] = {"ms": round(ms, 4), "tokens_per_s": round(batch / ms * 1e3, 1)}
            result["models"][label] = entry
        for kernel, ms, frac, of in _mixer_kernels(torch, virulix, sizes, pk, 2048, 8, 2048, flush, qwen):
            result["kernels"].append({"kernel": kernel, "ms": round(ms, 4), "frac": round(frac, 4), "of": of})
        print(json.dumps(result), flush=True)
        del virulix, qwen
        torch.cuda.empty_cache()


# --------------------------------------------------------------------------- Debisun beside Virulix
def _debisun_sizes(width, heads, kv_heads, dim, dense_ff, experts, identity, top, expert_ff, shared_ff, side, chunk, vocab):
    """Eight layers that use every mechanism of the design at one width."""
    mixer = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=dim ** -0.5, conv=4, softcap=30.0, bias_max=1024,
                 bias_rows=32, mask=dict(size=chunk))
    moe = dict(kind="moe", router=dict(experts=experts, identity=identity, top=top, scale=2.5), expert=dict(ff=expert_ff),
               shared=dict(ff=shared_ff))
    dense = dict(kind="dense", ff=dense_ff)
    layers = [dict(type="attention", mixer=mixer, mlp=mlp) for mlp in (dense, moe, moe, moe, moe, dense, dense, moe)]
    return dict(architecture="Debisun", vocab=vocab, width=width, norm=dict(eps=1e-6), token_side=dict(dim=side), layers=layers)


def _virulix_like(width, heads, kv_heads, dim, dense_ff, experts, top, expert_ff, shared_ff, vocab, **_):
    """Virulix with attention in every layer and the same order of dense and routed feed-forwards."""
    mixer = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=dim ** -0.5, q_temp=dict(coef=0.1, every=256))
    moe = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=expert_ff, limit=7.0),
               shared=dict(ff=shared_ff, limit=7.0))
    dense = dict(kind="dense", ff=dense_ff)
    layers = [dict(type="attention", mixer=mixer, mlp=mlp) for mlp in (dense, moe, moe, moe, moe, dense, dense, moe)]
    return dict(architecture="Virulix", vocab=vocab, width=width, norm=dict(eps=1e-6), layers=layers)


DEBISUN_SHAPES = {
    "2048": dict(width=2048, heads=16, kv_heads=4, dim=128, dense_ff=6144, experts=32, identity=4, top=4, expert_ff=768,
                 shared_ff=1536, side=64, chunk=1024, vocab=32768),
    "4096": dict(width=4096, heads=32, kv_heads=8, dim=128, dense_ff=12288, experts=64, identity=8, top=6, expert_ff=1024,
                 shared_ff=2048, side=128, chunk=1024, vocab=32768),
}


def _debisun_kernels(torch, debisun, virulix, sizes, pk, tokens_n, batch, context, flush):
    """The kernels of Debisun's mechanisms alone, each beside the like kernel of Virulix, with what the roofline
    allows: (name, ms, fraction of the measured peak, of what)."""
    from qwen_inference_lab_b200.cache import CacheManager
    from qwen_inference_lab_b200.engine import StepEntry, StepRunner
    from qwen_inference_lab_b200.kernels import ops
    from tests.harness import OnePartModel
    rows = []
    H, G, d, W = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["width"]
    tflops, gbs = pk["bf16_tflops"] * 1e12, pk["hbm_gbs"] * 1e9

    class Timer:
        def __init__(self):
            self.ms = []
        def __call__(self, fn):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            out = fn()
            stop.record()
            self.ms.append((start, stop))
            return out
        def median(self, skip):
            torch.cuda.synchronize()
            values = [a.elapsed_time(b) for a, b in self.ms[skip:]]
            self.ms = []
            return statistics.median(values)

    def measure(name, part, hidden, kernel_of, prompt_work, decode_bytes, stream_dtype=None):
        """``prompt_work``: (FLOPs, None) for a kernel bound by arithmetic, (None, bytes) for one bound by memory."""
        timer = Timer()
        shell = OnePartModel(part, hidden, torch.bfloat16, lambda ctx, x, view: kernel_of(ctx, x, view, timer))
        shell.stream_dtype = stream_dtype
        shell.inputs = torch.randn(4096, hidden, device="cuda").to(torch.bfloat16)
        pages = (batch + 1) * ((max(tokens_n, context) + PAGE_SIZE) // PAGE_SIZE + 2)
        cache = CacheManager(shell.cache_specs(), num_pages=pages, page_size=PAGE_SIZE, max_requests=batch + 1,
                             max_context=pages * PAGE_SIZE, dtype=torch.bfloat16, device="cuda")
        for g in cache.kv_groups:
            g.storage.normal_(0.0, 0.5)
        runner = StepRunner(shell, cache, max_step_tokens=tokens_n, use_graphs=False)
        ids = [i % 4096 for i in range(tokens_n)]
        for i in range(8):
            flush.zero_()
            cache.admit("p")
            runner.run([StepEntry("p", ids, [])])
            cache.release("p")
            shell.outputs.clear()
        ms = timer.median(3)
        flops, moved = prompt_work
        if flops is not None:
            rows.append((f"{name} prompt {tokens_n}", ms, flops / (ms * 1e-3) / tflops, "of the bf16 peak"))
        else:
            rows.append((f"{name} prompt {tokens_n}", ms, moved / (ms * 1e-3) / gbs, "of the copy bandwidth"))
        for rid in range(batch):
            cache.admit(rid)
            cache.ensure(rid, context)
            cache.advance(rid, context)
        for i in range(12):
            flush.zero_()
            runner.run([StepEntry(rid, [rid], []) for rid in range(batch)])
            shell.outputs.clear()
        ms = timer.median(4)
        rows.append((f"{name} decode b{batch} c{context}", ms, decode_bytes / (ms * 1e-3) / gbs, "of the copy bandwidth"))

    def attention_kernel(mixer):
        def kernel(ctx, x, view, timer):
            q = x[:, :H * d].contiguous()
            out = torch.empty_like(q)
            view = view[0] if isinstance(view, tuple) else view
            timer(lambda: mixer._attend(ctx, q, view, out))
            return out
        return kernel

    ours, theirs = debisun.layers[0].mixer, virulix.layers[0].mixer
    chunk = ours.chunk
    seen = lambda n: sum(min(i % chunk, i) + 1 for i in range(n)) if chunk else n * (n + 1) // 2      # (query, key) pairs
    decode_keys = lambda c: (c % chunk + 1) if chunk else c + 1
    measure("debisun attention (cap, distance table, chunks, sink)", ours, H * d, attention_kernel(ours),
            (4.0 * H * d * seen(tokens_n), None), batch * decode_keys(context) * 2 * G * d * 2)
    measure("virulix attention (distance slopes)", theirs, H * d, attention_kernel(theirs),
            (4.0 * H * d * tokens_n * (tokens_n + 1) / 2, None), batch * (context + 1) * 2 * G * d * 2)

    channels = (H + 2 * G) * d
    def conv_kernel(ctx, x, view, timer):
        qkv = x[:, :channels].contiguous()
        q = torch.empty((x.shape[0], H * d), dtype=x.dtype, device=x.device)
        pages_view, state = view
        timer(lambda: ops.short_conv_store(qkv, ours._conv_w, state.slots, q, pages_view.pages, ctx.positions, ctx.token_row,
                                           pages_view.block_table, ctx.seg_row, ctx.seg_start, ctx.seg_len, ctx.n_segments,
                                           H, G, d, d, pages_view.page_size))
        return q
    def store_kernel(ctx, x, view, timer):
        qkv = x[:, :channels].contiguous()
        q = torch.empty((x.shape[0], H * d), dtype=x.dtype, device=x.device)
        timer(lambda: ops.qkv_store(qkv, q, view.pages, ctx.positions, ctx.token_row, view.block_table, H, G, d, d,
                                    view.page_size, 0.1, 256))
        return q
    moved = lambda n: 2 * n * channels * 2          # every row read once and written once
    measure("debisun short convolution + page write", ours, channels, conv_kernel, (None, moved(tokens_n)), moved(batch))
    measure("virulix query temperature + page write", theirs, channels, store_kernel, (None, moved(tokens_n)), moved(batch))

    moe = next(l.feed_forward for l in debisun.layers if hasattr(l.feed_forward, "n_experts"))
    ff, E, top = moe.expert_size, moe.n_experts, moe.top
    def moe_kernel(ctx, x, view, timer):
        h = x[:, :W].contiguous()
        chosen, weights = ops.moe_route(h, moe.router.data, None, top, softmax_all=True, correction=moe.correction.data,
                                        weight_scale=moe.weight_scale)
        return timer(lambda: ops.moe_experts(h, chosen, weights, moe._up, None, moe._down, moe.activation, identity=True))
    measure("debisun routed experts (no gate matrix, identity outputs)", moe, W, moe_kernel,
            (2.0 * tokens_n * top * 2 * ff * W * E / (E + moe.identity), None), min(E, batch * top) * 2 * ff * W * 2)
    other = next(l.feed_forward for l in virulix.layers if hasattr(l.feed_forward, "n_experts"))
    def other_kernel(ctx, x, view, timer):
        h = x[:, :W].contiguous()
        chosen, weights = ops.moe_route(h, other.router.data, other.router_bias.data, other.top)
        return timer(lambda: ops.moe_experts(h, chosen, weights, other._gate, other._up, other._down, other.activation,
                                             limit=other.limit, alpha=other.alpha))
    measure("virulix routed experts (gated)", other, W, other_kernel, (2.0 * tokens_n * other.top * 3 * other.expert_size * W, None),
            min(other.n_experts, batch * other.top) * 3 * other.expert_size * W * 2)

    def ff_kernel(part):
        def kernel(ctx, x, view, timer):
            h = x[:, :W].contiguous()
            return timer(lambda: part.forward(ctx, h))
        return kernel
    dense = next(l.feed_forward for l in debisun.layers if hasattr(l.feed_forward, "up") and not hasattr(l.feed_forward, "n_experts"))
    inner = dense.intermediate_size
    measure("debisun feed-forward (squared relu)", dense, W, ff_kernel(dense), (2.0 * tokens_n * 2 * inner * W, None), 2 * inner * W * 2)
    gated = next(l.feed_forward for l in virulix.layers if hasattr(l.feed_forward, "gate_up"))
    measure("virulix feed-forward (gated gelu)", gated, W, ff_kernel(gated), (2.0 * tokens_n * 3 * inner * W, None), 3 * inner * W * 2)

    side = debisun.layers[0].after[0]
    def side_kernel(ctx, x, view, timer):
        stream = x[:, :W].float()
        return timer(lambda: side.forward(ctx, stream))
    # the stream is read and written in float32 and read once more in bfloat16; the two matrices are small
    side_bytes = lambda n: n * W * (4 + 4 + 4 + 2 + 2) + 2 * side.dim * W * 2
    measure("debisun token side input (5 kernels)", side, W, side_kernel, (None, side_bytes(tokens_n)), side_bytes(batch))
    return rows


def run_debisun(args):
    """Prefill and decode of Debisun at sizes like a real model's layers, beside Virulix (the engine's closest
    design: float32 stream, attention with a distance bias, routed experts with a shared one) of equal width, heads,
    layer count, feed-forward sizes and vocabulary, and the kernels of its mechanisms against their rooflines."""
    import torch
    from qwen_inference_lab_b200.config.model_config import DebisunConfig, VirulixConfig
    from qwen_inference_lab_b200.loading import random_model
    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for name in ([args.debisun_shape] if args.debisun_shape else sorted(DEBISUN_SHAPES)):
        sizes = DEBISUN_SHAPES[name]
        debisun = random_model(DebisunConfig.from_dict(_debisun_sizes(**sizes)), seed=0, device="cuda", dtype=torch.bfloat16)
        virulix = random_model(VirulixConfig.from_dict(_virulix_like(**sizes)), seed=0, device="cuda", dtype=torch.bfloat16)
        result = {"workload": "debisun", "width": sizes["width"], "layers": 8, "dtype": "bfloat16",
                  "peaks": "of measured" if pk["source"] == "measured" else "of fallback", "models": {}, "kernels": []}
        for label, model in (("debisun", debisun), ("virulix", virulix)):
            bench = _ModelBench(model, sizes["vocab"])
            entry = {}
            for tokens_n in (512, 2048):
                ms = bench.prefill(tokens_n, flush)
                entry[f"prefill_{tokens_n}"] = {"ms": round(ms, 3), "tokens_per_s": round(tokens_n / ms * 1e3, 1)}
            for batch, context in ((1, 2048), (8, 2048), (32, 2048)):
                ms = bench.decode(batch, context, args.steps, max(args.warmup, 6))
                entry[f"decode_b{batch}_c{context}"] = {"ms": round(ms, 4), "tokens_per_s": round(batch / ms * 1e3, 1)}
            result["models"][label] = entry
        for kernel, ms, frac, of in _debisun_kernels(torch, debisun, virulix, sizes, pk, 2048, 8, 2048 + 511, flush):
            result["kernels"].append({"kernel": kernel, "ms": round(ms, 4), "frac": round(frac, 4), "of": of})
        print(json.dumps(result), flush=True)
        del debisun, virulix
        torch.cuda.empty_cache()


# --------------------------------------------------------------------------- the reference
# --------------------------------------------------------------------------- Larolorn beside Virulix
def _larolorn_sizes(width, heads, kv_heads, dim, rank, rot, lin_heads, lin_dim, lin_vdim, ff, span, vocab):
    """Eight layers, latent attention and side-by-side mixers in turn; the third runs with the first one's tensors."""
    latent = dict(heads=heads, dim=dim, rot_dim=rot, vdim=dim, kv_rank=rank, scale=(dim + rot) ** -0.5,
                  rot=dict(base=10000.0, dims=rot), mask=dict(size=span))
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=dim ** -0.5, rot=dict(base=500000.0, dims=dim),
                mask=dict(size=span))
    right = dict(heads=lin_heads, dim=lin_dim, vdim=lin_vdim, decay=[1.0 - 2.0 ** -(2 + i % 8) for i in range(lin_heads)])
    mlp = dict(kind="dense", ff=ff, limit=7.0)
    one = dict(type="latent_attention", mixer=latent, mlp=mlp)
    two = dict(type="parallel", mixer=dict(left=left, right=right), mlp=mlp)
    layers = [one, two, dict(one, weights_of=0), two, one, two, one, two]
    return dict(architecture="Larolorn", vocab=vocab, width=width, norm=dict(eps=1e-6), residual_mult=0.5, logit_scale=0.25,
                layers=layers)


def _virulix_beside_larolorn(width, heads, kv_heads, dim, lin_heads, lin_dim, lin_vdim, ff, vocab, **_):
    """Virulix of equal width, heads, layer count, feed-forward size and vocabulary: attention and gated linear
    attention in turn, dense feed-forwards throughout."""
    attention = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=dim ** -0.5, q_temp=dict(coef=0.1, every=256))
    gla = dict(heads=lin_heads, dim=lin_dim, vdim=lin_vdim, tau=16.0, rank=16)
    mlp = dict(kind="dense", ff=ff)
    layers = [dict(type=kind, mixer=mixer, mlp=mlp) for kind, mixer in (("attention", attention), ("gla", gla)) * 4]
    return dict(architecture="Virulix", vocab=vocab, width=width, norm=dict(eps=1e-6), layers=layers)


LAROLORN_SHAPES = {
    "2048": dict(width=2048, heads=16, kv_heads=4, dim=128, rank=192, rot=64, lin_heads=8, lin_dim=128, lin_vdim=128, ff=6144,
                 span=1024, vocab=32768),
    "4096": dict(width=4096, heads=32, kv_heads=8, dim=128, rank=192, rot=64, lin_heads=16, lin_dim=128, lin_vdim=128, ff=12288,
                 span=1024, vocab=32768),
}


class _PartKernels:
    """Times one kernel (or a few) of a part inside the step function, on a whole prompt and on a step of single tokens
    behind ``context`` cached positions, an L2 flush before every step: rows of (name, ms, fraction, of what)."""

    def __init__(self, torch, pk, tokens_n, batch, context, flush):
        self.torch, self.tokens_n, self.batch, self.context, self.flush = torch, tokens_n, batch, context, flush
        self.tflops, self.gbs = pk["bf16_tflops"] * 1e12, pk["hbm_gbs"] * 1e9
        self.rows, self._marks = [], []

    def timed(self, fn):
        torch = self.torch
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # the device idles for a moment while the host queues what follows, so that the two events bracket the
        # kernels' time on the device and not the time the host takes to launch them
        torch.cuda._sleep(400_000)
        start.record()
        out = fn()
        stop.record()
        self._marks.append((start, stop))
        return out

    def _median(self, skip):
        self.torch.cuda.synchronize()
        values = [a.elapsed_time(b) for a, b in self._marks[skip:]]
        self._marks = []
        return statistics.median(values)

    def measure(self, name, part, hidden, kernel_of, prompt_work, decode_bytes, prompt_of=None):
        """``kernel_of(ctx, x, view)`` runs the kernel under ``self.timed``.  ``prompt_work``: (FLOPs, None) for a kernel
        bound by arithmetic, (None, bytes) for one bound by memory; ``prompt_of``: (peak in FLOP/s, its name) where
        the bound is not the bfloat16 tensor peak."""
        from qwen_inference_lab_b200.cache import CacheManager
        from qwen_inference_lab_b200.engine import StepEntry, StepRunner
        from tests.harness import OnePartModel
        torch, tokens_n, batch, context = self.torch, self.tokens_n, self.batch, self.context
        shell = OnePartModel(part, hidden, torch.bfloat16, kernel_of)
        shell.inputs = torch.randn(4096, hidden, device="cuda").to(torch.bfloat16)
        pages = (batch + 1) * ((max(tokens_n, context) + PAGE_SIZE) // PAGE_SIZE + 2)
        cache = CacheManager(shell.cache_specs(), num_pages=pages, page_size=PAGE_SIZE, max_requests=batch + 1,
                             max_context=pages * PAGE_SIZE, dtype=torch.bfloat16, device="cuda")
        for g in cache.kv_groups:
            g.storage.normal_(0.0, 0.5)
        runner = StepRunner(shell, cache, max_step_tokens=tokens_n, use_graphs=False)
        ids = [i % 4096 for i in range(tokens_n)]
        for i in range(8):
            self.flush.zero_()
            cache.admit("p")
            runner.run([StepEntry("p", ids, [])])
            cache.release("p")
            shell.outputs.clear()
        ms = self._median(3)
        flops, moved = prompt_work
        if flops is not None:
            peak, of = prompt_of or (self.tflops, "of the bf16 peak")
            self.rows.append((f"{name} prompt {tokens_n}", ms, flops / (ms * 1e-3) / peak, of))
        else:
            self.rows.append((f"{name} prompt {tokens_n}", ms, moved / (ms * 1e-3) / self.gbs, "of the copy bandwidth"))
        for rid in range(batch):
            cache.admit(rid)
            cache.ensure(rid, context)
            cache.advance(rid, context)
        for i in range(12):
            self.flush.zero_()
            runner.run([StepEntry(rid, [rid], []) for rid in range(batch)])
            shell.outputs.clear()
        ms = self._median(4)
        self.rows.append((f"{name} decode b{batch} c{context}", ms, decode_bytes / (ms * 1e-3) / self.gbs, "of the copy bandwidth"))


def _larolorn_kernels(torch, larolorn, virulix, sizes, pk, tokens_n, batch, context, flush):
    """The kernels of Larolorn's mechanisms alone, each beside the like kernel of Virulix, with what the roofline allows."""
    from qwen_inference_lab_b200.kernels import attention_mma, ops
    bench = _PartKernels(torch, pk, tokens_n, batch, context, flush)
    H, G, d, W = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["width"]
    span = sizes["span"]
    latent = next(l.mixer for l in larolorn.layers if hasattr(l.mixer, "latent_dim"))
    pair = next(l.mixer for l in larolorn.layers if hasattr(l.mixer, "left"))
    theirs = next(l.mixer for l in virulix.layers if hasattr(l.mixer, "plain_tail"))
    their_gla = next(l.mixer for l in virulix.layers if hasattr(l.mixer, "decay_rank"))
    pairs_window = sum(min(i, span - 1) + 1 for i in range(tokens_n))             # (query, key) pairs of a prompt
    pairs_chunk = sum(i % span + 1 for i in range(tokens_n))
    pairs_all = tokens_n * (tokens_n + 1) // 2

    # ---- attention itself
    row = latent.key_width
    def latent_attention(ctx, x, view):
        q = x[:, :H * row].contiguous()
        return bench.timed(lambda: latent.attend(ctx, q, view))
    bench.measure(f"larolorn latent attention (one key row of {row} for {H} heads, window)", latent, H * row, latent_attention,
                  (2.0 * H * (row + latent.latent_dim) * pairs_window, None), batch * min(context + 1, span) * row * 2)
    def grouped_attention(mixer):
        def kernel(ctx, x, view):
            q = x[:, :H * d].contiguous()
            out = torch.empty_like(q)
            view = view[0] if isinstance(view, tuple) else view
            bench.timed(lambda: mixer._attend(ctx, q, view, out))
            return out
        return kernel
    bench.measure("larolorn chunked attention (learned sinks)", pair.left, H * d, grouped_attention(pair.left),
                  (4.0 * H * d * pairs_chunk, None), batch * (context % span + 1) * 2 * G * d * 2)
    bench.measure("virulix attention (distance slopes)", theirs, H * d, grouped_attention(theirs),
                  (4.0 * H * d * pairs_all, None), batch * (context + 1) * 2 * G * d * 2)

    # ---- what stands between the projection and the attention
    channels = (H + 2 * G) * d
    moved = lambda n, width: 2 * n * width * 2          # every row read once and written once
    left = pair.left
    def rotate_store(ctx, x, view):
        qkv = x[:, :channels].contiguous()
        q = torch.empty((x.shape[0], H * d), dtype=x.dtype, device=x.device)
        bench.timed(lambda: ops.qk_rotate_store(qkv, (0, H * d, (H + G) * d), q, view.pages, left.whole_q_norm.data,
                                                left.whole_k_norm.data, left.whole_qk_norm_eps, left.position.freq,
                                                left.position.rotary_dim, left.position.layout, ctx.positions, ctx.token_row,
                                                view.block_table, H, G, d, d, view.page_size))
        return q
    def plain_store(ctx, x, view):
        qkv = x[:, :channels].contiguous()
        q = torch.empty((x.shape[0], H * d), dtype=x.dtype, device=x.device)
        bench.timed(lambda: ops.qkv_store(qkv, q, view.pages, ctx.positions, ctx.token_row, view.block_table, H, G, d, d,
                                          view.page_size, 0.1, 256))
        return q
    bench.measure("larolorn whole-projection norms + rotation + page write", left, channels, rotate_store,
                  (None, moved(tokens_n, channels)), moved(batch, channels))
    bench.measure("virulix query temperature + page write", theirs, channels, plain_store,
                  (None, moved(tokens_n, channels)), moved(batch, channels))
    q_in = H * (latent.plain_dim + latent.rot_dim)
    stacked = q_in + row + H
    def latent_tail(ctx, x, view):
        projected = x[:, :stacked].contiguous()
        return bench.timed(lambda: latent.prepare(ctx, projected, view))
    fold_flops = 2.0 * H * latent.plain_dim * latent.latent_dim
    bench.measure("larolorn latent norm + rotation + page write, queries through the key expansion", latent,
                  stacked, latent_tail, (fold_flops * tokens_n, None),
                  batch * (q_in + H * row) * 2 + H * latent.plain_dim * latent.latent_dim * 2)
    def latent_values(ctx, x, view):
        attended = x[:, :H * latent.value_width].contiguous()
        projected = x[:, :stacked].contiguous()
        return bench.timed(lambda: latent.expand(ctx, attended, projected))
    bench.measure("larolorn value expansion with the head gates", latent, max(stacked, H * latent.value_width), latent_values,
                  (2.0 * H * latent.value_dim * latent.latent_dim * tokens_n, None),
                  batch * H * (latent.value_width + latent.value_dim) * 2 + H * latent.value_dim * latent.latent_dim * 2)

    # ---- the recurrences: float32 on the CUDA cores by both designs, so the prompt's bound is the float32 FMA rate
    fma = (148 * 128 * 2 * 1.9e9, "of the float32 FMA rate (72 TFLOP/s nominal)")
    ours = pair.right
    oh, od, oe = ours.n_heads, ours.key_dim, ours.value_dim
    ours_width = ours.projection.out_features
    def decay_scan(ctx, x, view):
        projected = x[:, :ours_width].contiguous()
        view = view[-1] if isinstance(view, tuple) else view
        return bench.timed(lambda: ours.scan(ctx, projected, view))
    bench.measure("larolorn decayed linear attention scan", ours, ours_width, decay_scan, (5.0 * oh * od * oe * tokens_n, None),
                  batch * oh * od * oe * 4 * 2, prompt_of=fma)
    gh, gd, ge = their_gla.n_heads, their_gla.key_dim, their_gla.value_dim
    their_width = their_gla.projection.out_features
    def gla_scan(ctx, x, view):
        projected = x[:, :their_width].contiguous()
        mixed = torch.empty((x.shape[0], gh * ge), dtype=x.dtype, device=x.device)
        bench.timed(lambda: their_gla.scan(ctx, projected, view, mixed))
        return mixed
    bench.measure("virulix gated linear attention scan (decay per channel)", their_gla, max(their_width, 8), gla_scan,
                  (5.0 * gh * gd * ge * tokens_n, None), batch * gh * gd * ge * 4 * 2, prompt_of=fma)
    def whole_norm_gate(ctx, x, view):
        projected = x[:, :ours_width].contiguous()
        raw = projected[:, :oh * oe].float()
        mixed = torch.empty((x.shape[0], oh * oe), dtype=x.dtype, device=x.device)
        bench.timed(lambda: ops.lin_norm_gate_whole(raw, projected, ours.columns[3], ours.norm_weight.data, ours.norm_eps, mixed))
        return mixed
    gate_bytes = lambda n: n * oh * oe * (4 + 2 + 2)
    bench.measure("larolorn norm over all heads + gate", ours, ours_width, whole_norm_gate, (None, gate_bytes(tokens_n)),
                  gate_bytes(batch))

    # ---- joining the stream, and the feed-forwards
    def join(ctx, x, view):
        stream = x[:, :W].float()
        a, b = x[:, :W].float() * 3.0, x[:, :W].float() * 0.1
        weight = torch.ones(W, dtype=pair.left_weight.data.dtype, device=x.device)
        return bench.timed(lambda: ops.rms_join(stream, a, weight, 1e-6, 0.5, b=b, weight_a=pair.left_weight.data,
                                                weight_b=pair.right_weight.data, pre=0.5))
    join_bytes = lambda n: n * W * 4 * 4               # the stream read and written, two float32 branches read
    bench.measure("larolorn two normed branches join the stream (1 kernel)", latent, W, join, (None, join_bytes(tokens_n)),
                  join_bytes(batch))
    def feed_forward(part, **how):
        def kernel(ctx, x, view):
            h = x[:, :W].contiguous()
            return bench.timed(lambda: part.forward(ctx, h, **how))
        return kernel
    dense = next(l.feed_forward for l in larolorn.layers if l.feed_forward is not None)
    inner = dense.intermediate_size
    bench.measure("larolorn feed-forward (clamped, float32 result)", dense, W, feed_forward(dense, out_float32=True),
                  (2.0 * tokens_n * 3 * inner * W, None), 3 * inner * W * 2)
    gated = next(l.feed_forward for l in virulix.layers if hasattr(l.feed_forward, "gate_up"))
    bench.measure("virulix feed-forward (gated gelu)", gated, W, feed_forward(gated), (2.0 * tokens_n * 3 * inner * W, None),
                  3 * inner * W * 2)
    return bench.rows


def run_larolorn(args):
    """Prefill and decode of Larolorn at sizes like a real model's layers, beside Virulix (the engine's closest design:
    a float32 stream, attention layers and linear-attention layers with a float32 state) of equal width, heads, layer
    count, feed-forward size and vocabulary, and the kernels of its mechanisms against their rooflines."""
    import torch
    from qwen_inference_lab_b200.config.model_config import LarolornConfig, VirulixConfig
    from qwen_inference_lab_b200.loading import random_model
    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for name in ([args.larolorn_shape] if args.larolorn_shape else sorted(LAROLORN_SHAPES)):
        sizes = LAROLORN_SHAPES[name]
        larolorn = random_model(LarolornConfig.from_dict(_larolorn_sizes(**sizes)), seed=0, device="cuda", dtype=torch.bfloat16)
        virulix = random_model(VirulixConfig.from_dict(_virulix_beside_larolorn(**sizes)), seed=0, device="cuda", dtype=torch.bfloat16)
        result = {"workload": "larolorn", "width": sizes["width"], "layers": 8, "dtype": "bfloat16",
                  "peaks": "of measured" if pk["source"] == "measured" else "of fallback", "models": {}, "kernels": []}
        for label, model in (("larolorn", larolorn), ("virulix", virulix)):
            bench = _ModelBench(model, sizes["vocab"])
            entry = {}
            for tokens_n in (512, 2048):
                ms = bench.prefill(tokens_n, flush)
                entry[f"prefill_{tokens_n}"] = {"ms": round(ms, 3), "tokens_per_s": round(tokens_n / ms * 1e3, 1)}
            for batch, context in ((1, 2048), (8, 2048), (32, 2048)):
                ms = bench.decode(batch, context, args.steps, max(args.warmup, 6))
                entry[f"decode_b{batch}_c{context}"] = {"ms": round(ms, 4), "tokens_per_s": round(batch / ms * 1e3, 1)}
            result["models"][label] = entry
        for kernel, ms, frac, of in _larolorn_kernels(torch, larolorn, virulix, sizes, pk, 2048, 8, 2048 + 511, flush):
            result["kernels"].append({"kernel": kernel, "ms": round(ms, 4), "frac": round(frac, 4), "of": of})
        print(json.dumps(result), flush=True)
        del larolorn, virulix
        torch.cuda.empty_cache()


# --------------------------------------------------------------------------- Gogotar beside Larolorn
def _gogotar_sizes(width, heads, kv_heads, dim, rank, rot, ff, span, vocab, **_):
    """Six layers of which the middle two run twice (eight layer runs): latent attention with a dense feed-forward and
    chunked attention with routed experts in turn.  The latent's key row is as wide as Larolorn's (latent + rotated
    part there); an expert is a quarter of the dense feed-forward and a token uses four of thirty-two."""
    latent = dict(heads=heads, dim=dim, vdim=dim, kv_rank=rank + rot, q_rank=4 * (rank + rot), scale=dim ** -0.5)
    attention = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=dim ** -0.5, softcap=40.0, mask=dict(size=span),
                     rot=dict(base=1000000.0, dims=dim // 2, scaling=dict(factor=16.0, low=1.0, high=4.0, original=8192)))
    one = dict(type="latent_attention", mixer=latent, mlp=dict(kind="dense", ff=ff, limit=7.0))
    two = dict(type="attention", mixer=attention, mlp=dict(kind="moe", expert=dict(ff=ff // 4), router=dict(experts=32, top=4)))
    return dict(architecture="Gogotar", vocab=vocab, width=width, norm=dict(eps=1e-6), embedding=dict(scale=4.0),
                logit_softcap=25.0, loop=dict(start=2, stop=4, times=2), layers=[one, two, one, two, one, two])


def _gogotar_kernels(torch, gogotar, larolorn, sizes, pk, tokens_n, batch, context, flush):
    """The kernels of Gogotar's mechanisms alone, each beside the like kernel of Larolorn (of Virulix for the routed
    experts, which Larolorn has none of), with what the roofline allows."""
    from qwen_inference_lab_b200.kernels import ops
    from qwen_inference_lab_b200.parts import RoutedExperts
    bench = _PartKernels(torch, pk, tokens_n, batch, context, flush)
    H, G, d, W = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["width"]
    span = sizes["span"]
    ours_latent = next(l.mixer for l in gogotar.layers if hasattr(l.mixer, "latent_dim"))
    ours_attention = next(l.mixer for l in gogotar.layers if hasattr(l.mixer, "values_from_keys"))
    their_latent = next(l.mixer for l in larolorn.layers if hasattr(l.mixer, "latent_dim"))
    their_attention = next(l.mixer for l in larolorn.layers if hasattr(l.mixer, "left")).left
    pairs_window = sum(min(i, span - 1) + 1 for i in range(tokens_n))
    pairs_chunk = sum(i % span + 1 for i in range(tokens_n))
    pairs_all = tokens_n * (tokens_n + 1) // 2

    # ---- attention itself
    def latent_attention(latent):
        row = latent.key_width
        def kernel(ctx, x, view):
            q = x[:, :H * row].contiguous()
            return bench.timed(lambda: latent.attend(ctx, q, view))
        return kernel
    row = ours_latent.key_width
    bench.measure(f"gogotar latent attention (one key row of {row} for {H} heads, causal, sinks)", ours_latent, H * row,
                  latent_attention(ours_latent), (4.0 * H * row * pairs_all, None), batch * (context + 1) * row * 2)
    row = their_latent.key_width
    bench.measure(f"larolorn latent attention (one key row of {row}, window)", their_latent, H * row,
                  latent_attention(their_latent), (2.0 * H * (row + their_latent.latent_dim) * pairs_window, None),
                  batch * min(context + 1, span) * row * 2)
    def grouped_attention(mixer):
        def kernel(ctx, x, view):
            q = x[:, :H * d].contiguous()
            out = torch.empty_like(q)
            bench.timed(lambda: mixer._attend(ctx, q, view, out))
            return out
        return kernel
    for label, mixer in (("gogotar chunked attention (capped scores, learned sinks)", ours_attention),
                         ("larolorn chunked attention (learned sinks)", their_attention)):
        bench.measure(label, mixer, H * d, grouped_attention(mixer), (4.0 * H * d * pairs_chunk, None),
                      batch * (context % span + 1) * 2 * G * d * 2)

    # ---- what stands between the projection and the attention
    moved = lambda n, width: 2 * n * width * 2          # every row read once and written once
    def rotate_store(mixer, channels, per_head):
        q_weight, k_weight = (mixer.q_norm, mixer.k_norm) if per_head else (mixer.whole_q_norm, mixer.whole_k_norm)
        eps = mixer.qk_norm_eps if per_head else mixer.whole_qk_norm_eps
        def kernel(ctx, x, view):
            qkv = x[:, :channels].contiguous()
            q = torch.empty((x.shape[0], H * d), dtype=x.dtype, device=x.device)
            bench.timed(lambda: ops.qk_rotate_store(qkv, (0, H * d, H * d if per_head else (H + G) * d), q, view.pages,
                                                    q_weight.data, k_weight.data, eps, mixer.position.freq,
                                                    mixer.position.rotary_dim, mixer.position.layout, ctx.positions,
                                                    ctx.token_row, view.block_table, H, G, d, d, view.page_size,
                                                    per_head=per_head))
            return q
        return kernel
    channels = (H + G) * d
    bench.measure("gogotar per-head norms + rotation + page write (keys as values)", ours_attention, channels,
                  rotate_store(ours_attention, channels, True), (None, moved(tokens_n, channels) + tokens_n * G * d * 2),
                  moved(batch, channels))
    channels = (H + 2 * G) * d
    bench.measure("larolorn whole-projection norms + rotation + page write", their_attention, channels,
                  rotate_store(their_attention, channels, False), (None, moved(tokens_n, channels)), moved(batch, channels))
    def head_gates(ctx, x, view):
        attended = x[:, :H * d].contiguous()
        gates = x[:, :H].contiguous()
        return bench.timed(lambda: ops.head_gate(attended, d, gates, 0))
    bench.measure("gogotar gate per head on the attention's output", ours_attention, H * d, head_gates,
                  (None, moved(tokens_n, H * d)), moved(batch, H * d))
    stacked = ours_latent.projection.out_features
    def our_latent_tail(ctx, x, view):
        projected = x[:, :stacked].contiguous()
        return bench.timed(lambda: ours_latent.prepare(ctx, projected, view))
    fold = 2.0 * H * ours_latent.plain_dim * (ours_latent.latent_dim + ours_latent.query_latent)
    bench.measure("gogotar query latent norm + expansion, latent norm + page write, queries through the key expansion",
                  ours_latent, stacked, our_latent_tail, (fold * tokens_n, None),
                  batch * (stacked + H * ours_latent.key_width) * 2 + H * ours_latent.plain_dim * (ours_latent.latent_dim + ours_latent.query_latent) * 2)
    their_stacked = their_latent.projection.out_features
    def their_latent_tail(ctx, x, view):
        projected = x[:, :their_stacked].contiguous()
        return bench.timed(lambda: their_latent.prepare(ctx, projected, view))
    bench.measure("larolorn latent norm + rotation + page write, queries through the key expansion", their_latent,
                  their_stacked, their_latent_tail, (2.0 * H * their_latent.plain_dim * their_latent.latent_dim * tokens_n, None),
                  batch * (their_stacked + H * their_latent.key_width) * 2 + H * their_latent.plain_dim * their_latent.latent_dim * 2)
    def latent_values(latent, width):
        def kernel(ctx, x, view):
            attended = x[:, :H * latent.value_width].contiguous()
            projected = x[:, :width].contiguous()
            return bench.timed(lambda: latent.expand(ctx, attended, projected))
        return kernel
    for label, latent, width in (("gogotar value expansion with a gate per element", ours_latent, stacked),
                                 ("larolorn value expansion with the head gates", their_latent, their_stacked)):
        bench.measure(label, latent, max(width, H * latent.value_width), latent_values(latent, width),
                      (2.0 * H * latent.value_dim * latent.latent_dim * tokens_n, None),
                      batch * H * (latent.value_width + latent.value_dim) * 2 + H * latent.value_dim * latent.latent_dim * 2)

    # ---- joining the stream
    block = gogotar.layers[0]
    def norm_join(ctx, x, view):
        stream, branch = x[:, :W].float(), x[:, :W].float() * 3.0
        rows = torch.empty((x.shape[0], W), dtype=x.dtype, device=x.device)
        return bench.timed(lambda: ops.norm_join(stream, branch, block.post1.data, block.eps, "layer", next_weight=block.pre2.data,
                                                 rows=rows))
    join_bytes = lambda n: n * W * (4 * 3 + 2)           # the stream read and written, a float32 branch read, rows written
    bench.measure("gogotar a layer-normed branch joins the stream, the next layer norm behind it (1 kernel)", ours_latent, W,
                  norm_join, (None, join_bytes(tokens_n)), join_bytes(batch))
    their_block = larolorn.layers[0]
    def rms_join(ctx, x, view):
        stream, branch = x[:, :W].float(), x[:, :W].float() * 3.0
        rows = torch.empty((x.shape[0], W), dtype=x.dtype, device=x.device)
        return bench.timed(lambda: ops.rms_join(stream, branch, their_block.mixer_norm.data, their_block.eps, 0.5, rows=rows))
    bench.measure("larolorn a normed branch joins the stream, its rounded copy behind it (1 kernel)", their_latent, W,
                  rms_join, (None, join_bytes(tokens_n)), join_bytes(batch))

    # ---- routed experts, beside routed experts that renormalise the chosen logits (Virulix's)
    def feed_forward(part, **how):
        def kernel(ctx, x, view):
            h = x[:, :W].contiguous()
            return bench.timed(lambda: part.forward(ctx, h, **how))
        return kernel
    ours = next(l.feed_forward for l in gogotar.layers if hasattr(l.feed_forward, "n_experts"))
    names = dict(router="r", router_bias=None, expert=lambda index, which: f"e{index}.{which}")
    theirs = RoutedExperts(W, ours.expert_size, ours.n_experts, ours.top, names=names, activation="silu")
    for param in theirs.all_named_params().values():
        param.data = (torch.randn(param.shape, device="cuda") * 0.02).to(torch.bfloat16)
    theirs.finalize(torch.device("cuda"), torch.bfloat16)
    active = 3 * ours.expert_size * W
    touched = lambda n: min(ours.n_experts, n * ours.top) * active * 2
    bench.measure("gogotar routed experts (softmax over all, unrenormalised, float32 result)", ours, W,
                  feed_forward(ours, out_float32=True), (2.0 * tokens_n * ours.top * active, None), touched(batch))
    bench.measure("virulix-style routed experts (softmax over the chosen)", theirs, W, feed_forward(theirs),
                  (2.0 * tokens_n * ours.top * active, None), touched(batch))
    return bench.rows


def run_gogotar(args):
    """Prefill and decode of Gogotar at sizes like a real model's layers, beside Larolorn (the engine's closest design: a
    float32 stream, latent attention, chunked attention with learned sinks, clamped feed-forwards, branches normed on
    their way into the stream) of equal width, heads, layer runs, key row, feed-forward size and vocabulary, and the
    kernels of its mechanisms against their rooflines."""
    import torch
    from qwen_inference_lab_b200.config.model_config import GogotarConfig, LarolornConfig
    from qwen_inference_lab_b200.loading import random_model
    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for name in ([args.gogotar_shape] if args.gogotar_shape else sorted(LAROLORN_SHAPES)):
        sizes = LAROLORN_SHAPES[name]
        gogotar = random_model(GogotarConfig.from_dict(_gogotar_sizes(**sizes)), seed=0, device="cuda", dtype=torch.bfloat16)
        larolorn = random_model(LarolornConfig.from_dict(_larolorn_sizes(**sizes)), seed=0, device="cuda", dtype=torch.bfloat16)
        result = {"workload": "gogotar", "width": sizes["width"], "layer_runs": 8, "dtype": "bfloat16",
                  "peaks": "of measured" if pk["source"] == "measured" else "of fallback", "models": {}, "kernels": []}
        for label, model in (("gogotar", gogotar), ("larolorn", larolorn)):
            bench = _ModelBench(model, sizes["vocab"])
            entry = {}
            for tokens_n in (512, 2048):
                ms = bench.prefill(tokens_n, flush)
                entry[f"prefill_{tokens_n}"] = {"ms": round(ms, 3), "tokens_per_s": round(tokens_n / ms * 1e3, 1)}
            for batch, context in ((1, 2048), (8, 2048), (32, 2048)):
                ms = bench.decode(batch, context, args.steps, max(args.warmup, 6))
                entry[f"decode_b{batch}_c{context}"] = {"ms": round(ms, 4), "tokens_per_s": round(batch / ms * 1e3, 1)}
            result["models"][label] = entry
        for kernel, ms, frac, of in _gogotar_kernels(torch, gogotar, larolorn, sizes, pk, 2048, 8, 2048 + 511, flush):
            result["kernels"].append({"kernel": kernel, "ms": round(ms, 4), "frac": round(frac, 4), "of": of})
        print(json.dumps(result), flush=True)
        del gogotar, larolorn
        torch.cuda.empty_cache()


def run_reference(args):
    ref = ROOT / "baseline" / "_ref"
    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        return 0
    if not (ref / "qil" / "engine.py").is_file():
        return unavailable("the reference is not installed under baseline/_ref")
    sys.path.insert(0, str(ref))
    try:
        import torch
        from qil.config import ModelConfig
        from qil.engine import Engine
        from qil.model import Qwen3
    except Exception as error:  # noqa: BLE001
        return unavailable(f"import failed: {type(error).__name__}: {error}")
    batch = args.batch
    fields = ModelConfig.__dataclass_fields__
    config = ModelConfig(**{k: v for k, v in QWEN3_8B.items() if k in fields})
    try:
        torch.manual_seed(0)
        with torch.device("cuda"):
            model = Qwen3(config).to(dtype=torch.bfloat16).eval()
        with torch.no_grad():
            for parameter in model.parameters():
                if parameter.ndim == 2:
                    parameter.normal_(0.0, 0.02)
        new_tokens = args.steps + args.warmup + 4
        prompt_len = CONTEXT - 1
        pages = batch * ((prompt_len + new_tokens + PAGE_SIZE - 1) // PAGE_SIZE + 1)
        engine = Engine(model, num_pages=pages, page_size=PAGE_SIZE, token_budget=2048, prefill_chunk=2048,
                        max_active=batch, decode_attention="paged")
        generator = torch.Generator().manual_seed(3)
        for _ in range(batch):
            prompt = torch.randint(0, config.vocab_size, (prompt_len,), generator=generator).tolist()
            engine.submit(prompt, max_new_tokens=new_tokens, ignore_eos=True)
        while any(r.computed < len(r.prompt) for r in engine.scheduler.requests.values()):
            engine.step()
        for _ in range(args.warmup):
            engine.step()
        torch.cuda.synchronize()
        with ClockSampler() as sampler:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin = time.perf_counter()
            start.record()
            emitted = 0
            for _ in range(args.steps):
                emitted += len(engine.step())
            stop.record()
            torch.cuda.synchronize()
            elapsed = time.perf_counter() - begin
        ms = start.elapsed_time(stop) / args.steps
    except Exception as error:  # noqa: BLE001
        return unavailable(f"the reference failed on this configuration: {type(error).__name__}: {str(error)[:200]}")
    pk = peaks()
    achieved = decode_bytes(QWEN3_8B, batch, CONTEXT) / (ms * 1e-3) / 1e9
    of = "of measured" if pk["source"] == "measured" else "of fallback"
    # What the reference copies per decode step (qil/model.py:143-152, qil/cache.py:103-131, qil/engine.py:96-100):
    # it builds int64 tensors from Python lists for the token ids, the positions (lengths derive from them on the
    # device), the write slots and the padded page table, and reads back one flag and the chosen ids.
    table_width = (CONTEXT + args.warmup + args.steps + PAGE_SIZE - 1) // PAGE_SIZE
    h2d = 8 * (batch + batch + batch + batch * table_width)
    d2h = 1 + 8 * batch
    print(json.dumps({
        "metric": "decode tokens/s (Qwen3-8B shape, batch 8, context 8192)", "impl": "reference",
        "value": round(batch / ms * 1e3, 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights, random token ids",
        "config": config_record(QWEN3_8B, "Qwen3-8B shape", batch, CONTEXT, QWEN3_8B["num_hidden_layers"], of),
        "clocks": sampler.summary(),
        "e2e": {"value": round(emitted / elapsed, 2), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(elapsed / args.steps * 1e3, 2)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }), flush=True)
    return 0


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=32)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    parser.add_argument("--quick", action="store_true", help="skip the batch 1 and 64 points")
    parser.add_argument("--only", choices=["decode", "prefill", "mixed", "virulix", "debisun", "larolorn", "gogotar"], default=None,
                        help="run just this part and print its result instead of the JSON line; mixed = 64 requests "
                             "with prompts of 16 to 2048 tokens and 128 new tokens each through Engine.generate; "
                             "virulix = the Virulix design beside dense Qwen3 of equal size, and its mixers' kernels; "
                             "debisun = the Debisun design beside Virulix of equal size, and its mechanisms' kernels; "
                             "larolorn = the Larolorn design beside Virulix of equal size, and its mechanisms' kernels; "
                             "gogotar = the Gogotar design beside Larolorn of equal size, and its mechanisms' kernels")
    parser.add_argument("--virulix-shape", choices=sorted(VIRULIX_SHAPES), default=None,
                        help="width of --only virulix (default: all)")
    parser.add_argument("--debisun-shape", choices=sorted(DEBISUN_SHAPES), default=None,
                        help="width of --only debisun (default: all)")
    parser.add_argument("--larolorn-shape", choices=sorted(LAROLORN_SHAPES), default=None,
                        help="width of --only larolorn (default: all)")
    parser.add_argument("--gogotar-shape", choices=sorted(LAROLORN_SHAPES), default=None,
                        help="width of --only gogotar (default: all)")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="8b", help="layer sizes (default: Qwen3-8B)")
    parser.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    parser.add_argument("--context", type=int, default=CONTEXT, help="cached tokens per request (profiling aid)")
    parser.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                        help="prompt length of --only prefill (the JSON line always uses 2048)")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args)
    if args.only == "larolorn":
        run_larolorn(args)
        return
    if args.only == "gogotar":
        run_gogotar(args)
        return 0
    if args.only == "debisun":
        run_debisun(args)
        return 0
    if args.only == "virulix":
        run_virulix(args)
        return 0
    run_ours(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
