#!/usr/bin/env python3
"""Benchmark of the engine's decode step on one B200: ``python bench.py --gpus 1 --steps K --warmup W``.

The model has the layer sizes of the MiniCPM-2B shape (40 layers, hidden 2304, 36/36 heads of
64, intermediate 5760, vocabulary 122753, tied embeddings) with random bfloat16 weights made
on the device.  A step is one decode step of a batch of 8 requests whose caches hold about
4096 tokens each (synthetic cache contents: decoding cost does not depend on the values).

One JSON line is printed:
  value       decoded tokens per second, device-timed (CUDA events around K steps of the engine's
              step function + the sampling kernel; token ids are fixed, nothing is read back);
  e2e         the same through the Python entry point (``batch_infer_one_round``): every step copies
              its token ids and block tables from pinned host memory and reads the sampled ids back;
  prefill     one 2,048-token prompt through the step function;
  roofline    bytes a decode step must read (every weight once + the live requests' cache) / time;
  points      decode tokens per second at batch 1 and 64 (context 4096) and at context 512;
  plain       the same engine run one call per operator with library products, the plain attention kernel, separate norm
              kernels and no CUDA graphs: the shape of the reference's step (src/models/jiuge/jiuge.cpp:195-258), which
              cannot itself be built here; ``vs_baseline`` is ``value`` over this path's batch-8 decode rate;
  kernels     device time of each dominant kernel alone at the benchmark's shape (one launch record of the model at a time,
              walking through the layers so that weights and cache come from memory, not from L2) with its achieved
              GB/s or TFLOP/s over the measured peak.
Peaks come from MEASURED_PEAKS.json beside this file if present, else from the fallback values.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# configs[2] of the benchmark definition: the MiniCPM-2B shape
SHAPE_2B = dict(model_type="minicpm", num_hidden_layers=40, hidden_size=2304, num_attention_heads=36,
                num_key_value_heads=36, intermediate_size=5760, vocab_size=122753,
                max_position_embeddings=4096, rms_norm_eps=1e-5, rope_theta=10000.0, scale_emb=12,
                scale_depth=1.4, dim_model_base=256, tie_word_embeddings=True)
# configs[3] and configs[4]: the shapes of the two serving-style workloads (--workload)
SHAPE_1B = dict(model_type="minicpm", num_hidden_layers=52, hidden_size=1536, num_attention_heads=24,
                num_key_value_heads=8, intermediate_size=3840, vocab_size=73440,
                max_position_embeddings=4096, rms_norm_eps=1e-5, rope_theta=10000.0, scale_emb=12,
                scale_depth=1.4, dim_model_base=256, tie_word_embeddings=True)
SHAPE_8B = dict(model_type="fm9g", num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
                num_key_value_heads=2, intermediate_size=16384, vocab_size=73448,
                max_position_embeddings=4096, rms_norm_eps=1e-5, rope_theta=10000.0, scale_emb=12,
                scale_depth=1.4, dim_model_base=256, tie_word_embeddings=False)
WORKLOADS = {
    # name: (shape, requests, prompt lengths, new tokens, portion size, token budget of a step)
    "1b-mixed": (SHAPE_1B, 32, (16, 1024), 128, 256, 512),
    "8b-serving": (SHAPE_8B, 64, (512, 2048), 256, 512, 2048),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                data = json.load(f)
            flat = {}
            def walk(d):
                for k, v in d.items():
                    if isinstance(v, dict):
                        walk(v)
                    elif isinstance(v, (int, float)):
                        flat.setdefault(k, float(v))
            walk(data)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return {"hbm_gbs": flat["hbm_gbs"], "bf16_tflops": flat["bf16_tflops"],
                        "bf16_tflops_sustained": flat.get("bf16_tflops_sustained", flat["bf16_tflops"])}, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi in the background while the timed region runs; stopped by its own PID."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __enter__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()

    def summary(self):
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def run_workload(name, layers=None):
    """A serving-style workload through the scheduler: all requests are submitted at once, prompts are
    cut into portions under the step's token budget beside the others' decoded tokens, every request
    generates its full count (no stop token).  Prints one JSON line of its own kind."""
    import random
    import torch
    from infinicore_infer_b200.config import MiniCPMConfig
    from infinicore_infer_b200.engine import Engine, Generator
    from infinicore_infer_b200.parts import model_manifest
    from infinicore_infer_b200.weights import DeviceRandomWeights

    shape, n_req, (lo, hi), new_tokens, chunk, budget = WORKLOADS[name]
    shape = dict(shape)
    full_layers = shape["num_hidden_layers"]
    if layers:
        shape["num_hidden_layers"] = layers
    cfg = MiniCPMConfig.from_dict(shape)
    spec = cfg.model_spec()
    dev, page = "cuda:0", 16
    rng = random.Random(0)
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(rng.randint(lo, hi))] for _ in range(n_req)]
    cache_tokens = sum(len(p) + new_tokens + page for p in prompts)
    weights = DeviceRandomWeights(model_manifest(spec), seed=0, compute_dtype=torch.bfloat16, device=dev, std=0.02,
                                  untied=not shape["tie_word_embeddings"])
    engine = Engine(spec, weights, dtype=torch.bfloat16, device=dev, cache_tokens=cache_tokens, page_size=page,
                    max_requests=n_req, max_step_tokens=budget)
    results = []
    with ClockSampler() as clocks:
        for rep in range(2):                   # the first pass warms up (graph captures, lazy handles)
            g = Generator(engine, max_batch=n_req, max_tokens_per_step=budget, chunk_size=chunk)
            reqs = [g.submit(p, max_new_tokens=new_tokens, eos_token_ids=()) for p in prompts]
            torch.cuda.synchronize()
            l0 = engine.kernel_launches
            t0 = time.perf_counter()
            g.run()
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            generated = sum(len(r.generated) for r in reqs)
            results.append((dt, generated, dict(g.scheduler.counters), engine.kernel_launches - l0))
    dt, generated, counters, launches = results[-1]
    prompt_tokens = sum(len(p) for p in prompts)
    print(json.dumps({
        "workload": name, "metric": "generated tok/s through the scheduler (host tokens in and out every step)",
        "value": round(generated / dt, 1), "unit": "tokens/s", "seconds": round(dt, 3),
        "generated_tokens": generated, "prompt_tokens": prompt_tokens,
        "all_tokens_per_s": round((generated + prompt_tokens) / dt, 1),
        "scheduler": counters, "gpu_launches": int(launches), "dtype": "bf16",
        "data": "synthetic: random-init weights N(0,0.02), uniform random token ids",
        "config": {"model": name, "layers": cfg.num_hidden_layers, "layers_of_shape": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "requests": n_req, "prompt_len_min": lo, "prompt_len_max": hi, "new_tokens": new_tokens,
                   "portion": chunk, "tokens_per_step": budget, "page_size": page},
        "clocks": clocks.summary(),
    }))
    return 0



def time_records(engine, ctx, which, repeats=3):
    """Device time (microseconds per launch) of one kind of launch record, run alone: ``which(l)`` gives the index of
    layer l's record (or None to skip the layer).  The records of all layers run one after the other as one CUDA graph,
    so each launch reads its own layer's weights and cache pages from memory and follows its predecessor as closely as
    in a step; the best of ``repeats`` replays counts."""
    import ctypes
    import torch
    from infinicore_infer_b200 import kernels
    from infinicore_infer_b200.parts.program import SLOT, RunnerStep
    runner, prog = engine.runner, engine.program
    T = ctx.ntok
    logits = torch.empty(max(1, ctx.want_rows.numel()), engine.spec.vocab_size, dtype=torch.float32, device=engine.device)
    runner.buffers.slot[SLOT["logits"]] = logits.data_ptr()
    runner.buffers.bytes[SLOT["logits"]] = logits.numel() * 4
    step = RunnerStep(ntok=T, nreq=ctx.nreq, n_want=ctx.want_rows.numel(), context=ctx.context, tokens=ctx.tokens.data_ptr(),
                      positions=ctx.positions.data_ptr(), row_req=ctx.row_req.data_ptr(), req_start=ctx.req_start.data_ptr(),
                      req_pos=ctx.req_pos.data_ptr(), want_rows=ctx.want_rows.data_ptr())
    for g, table in enumerate(ctx.block_tables):
        step.block_tables[g] = table.data_ptr()
    for name, index in prog.lists.items():
        view, n = ctx.lists[name]
        step.lists[index] = view.data_ptr() if view is not None else None
        step.list_n[index] = n
    indices = [i for i in (which(l) for l in range(len(engine.spec.order))) if i is not None]

    def walk():
        stream = kernels._stream()          # asked for at each walk: a capture runs on a stream of its own
        for i in indices:
            rc = runner.lib.jk_runner_run(ctypes.byref(runner.env), prog.ops, i, 1, ctypes.byref(step), ctypes.byref(runner.buffers), 1, stream)
            if rc:
                raise RuntimeError(runner.lib.jk_runner_last_error().decode())
    walk()
    torch.cuda.synchronize()
    # the walk as one CUDA graph: launches follow one another as they do in a step (each starts under the tail of the one
    # before), without the host's time between them
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        walk()
    graph.replay()
    torch.cuda.synchronize()
    best = None
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1000.0 / len(indices)
        best = us if best is None else min(best, us)
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the shape has (both numbers are reported)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 and context 512 points")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-context-buckets", action="store_true", help="plan every decode step for the model's longest context")
    ap.add_argument("--no-plain", action="store_true", help="skip the plain (one call per operator) baseline")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel timings")
    ap.add_argument("--profile", default=None, choices=["decode", "prefill"],
                    help="run a few steps between cudaProfilerStart/Stop (for ncu --profile-from-start off) and exit")
    ap.add_argument("--shape", default="2b", choices=["2b", "1b", "8b"],
                    help="layer sizes: 2b is the headline configuration; the others are for profiles and side measurements")
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="instead of the decode benchmark: a serving-style workload through the scheduler")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "InfiniCore-Infer has no Python package to install (xmake C++ project) and its device "
                          "libraries infiniop/infinirt/infiniccl are absent; it cannot be built or run here"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported, run with --gpus 1")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.workload:
        return run_workload(args.workload, args.layers)

    import torch
    from infinicore_infer_b200.config import MiniCPMConfig
    from infinicore_infer_b200.engine import Engine, StepEntry
    from infinicore_infer_b200.jiuge import JiugeForCauslLM
    from infinicore_infer_b200.parts import model_manifest
    from infinicore_infer_b200.tasks import InferTask, KVCache
    from infinicore_infer_b200.weights import DeviceRandomWeights
    from infinicore_infer_b200 import kernels

    peaks, peak_source = load_peaks()
    shape = dict({"2b": SHAPE_2B, "1b": SHAPE_1B, "8b": SHAPE_8B}[args.shape])
    shape_name = {"2b": "MiniCPM-2B shape", "1b": "MiniCPM-1B shape", "8b": "FM9G-8B-class shape"}[args.shape]
    full_layers = shape["num_hidden_layers"]
    if args.layers:
        shape["num_hidden_layers"] = args.layers
    shape["max_position_embeddings"] = max(args.context, 4096)
    cfg = MiniCPMConfig.from_dict(shape)
    spec = cfg.model_spec()
    dev = "cuda:0"
    page = 16
    max_b = 1 if args.no_points else 64
    max_b = max(max_b, args.batch)
    cache_tokens = max(max_b * (args.context + page), 2048 + 4 * page)      # the decode points, or the prompt of 2,048 tokens
    t_load = time.time()
    weights = DeviceRandomWeights(model_manifest(spec), seed=0, compute_dtype=torch.bfloat16, device=dev, std=0.02,
                                  untied=not shape["tie_word_embeddings"])
    engine = Engine(spec, weights, dtype=torch.bfloat16, device=dev, cache_tokens=cache_tokens, page_size=page,
                    max_requests=max_b, max_step_tokens=4096, context_buckets=not args.no_context_buckets)
    engine.config = cfg
    for view in engine.cache.views:          # synthetic cache contents
        view.k_pages.normal_(0, 0.5)
        view.v_pages.normal_(0, 0.5)
    torch.cuda.synchronize()
    t_load = time.time() - t_load
    model = JiugeForCauslLM.from_engine(engine)
    V = spec.vocab_size
    gen = torch.Generator().manual_seed(0)
    kv_bytes_per_token = sum(2 * v.k_pages.shape[1] * v.k_pages.shape[3] * v.k_pages.element_size()
                             for v in engine.cache.views)
    weight_bytes = engine.model.weight_bytes_per_step()

    def fill(n_req, length, prefix):
        """n_req requests whose caches hold ``length`` positions (contents are the synthetic values)."""
        ids = []
        for i in range(n_req):
            rid = f"{prefix}{i}"
            engine.begin(rid)
            engine.cache.reserve(rid, length)
            engine.cache.commit(rid, length)
            ids.append(rid)
        return ids

    def drop(ids):
        for rid in ids:
            engine.end(rid)

    def decode_device(n_req, context, steps, warmup):
        """Device time of ``steps`` decode steps (step function + argmax) with fixed token ids."""
        start = context - (steps + warmup) - 1
        ids = fill(n_req, start, "d")
        toks = torch.randint(0, V, (n_req,), generator=gen).tolist()
        out = torch.empty(n_req, dtype=torch.int32, device=dev)
        entries = [StepEntry(r, [t], [0]) for r, t in zip(ids, toks)]
        for _ in range(warmup):
            kernels.argmax(engine.step(entries), out)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = engine.kernel_launches
        e0.record()
        for _ in range(steps):
            kernels.argmax(engine.step(entries), out)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        launches = engine.kernel_launches - l0 + steps
        mean_ctx = start + warmup + (steps + 1) / 2
        drop(ids)
        return ms, launches, mean_ctx

    def decode_e2e(n_req, context, steps, warmup):
        """The same through ``batch_infer_one_round``: host token ids in, sampled ids out, every step."""
        start = context - (steps + warmup) - 1
        tasks = []
        for i in range(n_req):
            t = InferTask(i, [int(torch.randint(0, V, (1,), generator=gen))], context + 8, 0.0, 1, 1.0, [])
            kv = KVCache(model)
            engine.cache.reserve(kv.data(), start)
            engine.cache.commit(kv.data(), start)
            t.bind_kvcache(kv)
            t.pos = start
            tasks.append(t)
        for _ in range(warmup):
            for t, tok in zip(tasks, model.batch_infer_one_round(tasks)):
                t.next(tok)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.perf_counter()
        e0.record()
        for _ in range(steps):
            for t, tok in zip(tasks, model.batch_infer_one_round(tasks)):
                t.next(tok)
        e1.record()
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - w0) * 1000 / steps
        ms = max(e0.elapsed_time(e1) / steps, wall_ms)
        for t in tasks:
            t.kvcache().drop(model)
        return ms

    if args.profile:
        if args.profile == "decode":
            ids = fill(args.batch, args.context - 16, "q")
            entries = [StepEntry(r, [1], [0]) for r in ids]
            out = torch.empty(args.batch, dtype=torch.int32, device=dev)
            for _ in range(3):
                kernels.argmax(engine.step(entries), out)
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            for _ in range(2):
                kernels.argmax(engine.step(entries), out)
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        else:
            ptoks = torch.randint(0, V, (2048,), generator=gen).tolist()
            engine.step([StepEntry("w", ptoks, [2047])]); engine.end("w")
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            engine.step([StepEntry("w", ptoks, [2047])])
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        print(json.dumps({"profiled": args.profile, "layers": cfg.num_hidden_layers}))
        return 0

    result_points = {}
    with ClockSampler() as clocks:
        ms, launches, mean_ctx = decode_device(args.batch, args.context, args.steps, args.warmup)
        e2e_ms = decode_e2e(args.batch, args.context, args.steps, args.warmup)
    clock_summary = clocks.summary()
    value = args.batch * 1000.0 / ms
    step_bytes = weight_bytes + args.batch * mean_ctx * kv_bytes_per_token
    achieved = step_bytes / (ms * 1e-3) / 1e9

    prefill = None
    if not args.no_prefill:
        T = 2048
        ptoks = torch.randint(0, V, (T,), generator=gen).tolist()
        times = []
        for i in range(4):
            rid = f"p{i}"
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine.step([StepEntry(rid, ptoks, [T - 1])])
            e1.record()
            torch.cuda.synchronize()
            engine.end(rid)
            if i >= 1:
                times.append(e0.elapsed_time(e1))
        pms = min(times)
        L, d, nh, dh, di = cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.head_dim, cfg.intermediate_size
        nkv = cfg.num_key_value_heads
        per_tok = 2 * L * (d * (nh + 2 * nkv) * dh + nh * dh * d + 3 * d * di)
        flops = T * per_tok + L * 2 * T * T * dh * nh + 2 * d * V
        prefill = {"value": round(T * 1000.0 / pms, 1), "tokens": T, "ms": round(pms, 3),
                   "frac": round(flops / (pms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4),
                   "frac_of_sustained": round(flops / (pms * 1e-3) / (peaks["bf16_tflops_sustained"] * 1e12), 4),
                   "tflops": round(flops / (pms * 1e-3) / 1e12, 1), "peak_source": peak_source}

    if not args.no_points:
        psteps, pwarm = min(args.steps, 32), 4
        for name, b, c in (("decode_b1", 1, args.context), ("decode_b64", 64, args.context),
                           ("decode_b1_ctx512", 1, 512), ("decode_b8_ctx512", 8, 512), ("decode_b64_ctx512", 64, 512)):
            pm = sorted(decode_device(b, c, psteps, pwarm)[0] for _ in range(3))[1]       # the median of three runs
            result_points[name] = round(b * 1000.0 / pm, 1)

    # ---- each dominant kernel alone ---------------------------------------------------------------------------
    kernel_block = None
    if not args.no_kernels:
        L, d, nh, nkv, dh, di = (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                                 cfg.head_dim, cfg.intermediate_size)
        nq = (nh + 2 * nkv) * dh
        rec = lambda k: (lambda l: 1 + 7 * l + k)             # a layer's records: norm, qkv, attention, o, norm, gate/up, down
        last = 1 + 7 * L + 1                                   # the output product
        kernel_block = {"peak_hbm_gbs": peaks["hbm_gbs"], "peak_bf16_tflops": peaks["bf16_tflops"], "peak_source": peak_source}

        def mem(name, us, nbytes):
            gbs = nbytes / (us * 1e-6) / 1e9
            kernel_block.update({f"{name}_us": round(us, 2), f"{name}_gbs": round(gbs, 1), f"{name}_frac": round(gbs / peaks["hbm_gbs"], 3)})

        def flop(name, us, flops):
            tf = flops / (us * 1e-6) / 1e12
            kernel_block.update({f"{name}_us": round(us, 2), f"{name}_tflops": round(tf, 1), f"{name}_frac": round(tf / peaks["bf16_tflops"], 3)})

        ids = fill(args.batch, args.context - 2, "k")
        entries = [StepEntry(r, [1], [0]) for r in ids]
        for r in ids:
            engine.cache.reserve(r, args.context - 1)
        dctx = engine._upload(entries, [args.context - 2] * args.batch, args.batch, args.batch)
        mem("decode_qkv", time_records(engine, dctx, rec(1)), nq * d * 2)
        mem("decode_attention", time_records(engine, dctx, rec(2)), args.batch * (args.context - 1) * kv_bytes_per_token / L)
        mem("decode_o", time_records(engine, dctx, rec(3)), d * nh * dh * 2)
        mem("decode_gate_up", time_records(engine, dctx, rec(5)), 2 * di * d * 2)
        mem("decode_down", time_records(engine, dctx, rec(6)), d * di * 2)
        mem("decode_lm_head", time_records(engine, dctx, lambda l: last if l < 3 else None), V * d * 2)
        layer_bytes = (nq * d + d * nh * dh + 3 * di * d) * 2
        layer_us = sum(kernel_block[f"decode_{k}_us"] for k in ("qkv", "o", "gate_up", "down"))
        kernel_block["decode_layer_products_us"] = round(layer_us, 2)
        kernel_block["decode_layer_products_frac"] = round(layer_bytes / (layer_us * 1e-6) / 1e9 / peaks["hbm_gbs"], 3)
        drop(ids)
        T = 2048
        ptoks = torch.randint(0, V, (T,), generator=gen).tolist()
        engine.begin("kp")
        engine.cache.reserve("kp", T)
        pctx = engine._upload([StepEntry("kp", ptoks, [T - 1])], [0], 1, T)
        flop("prefill_qkv", time_records(engine, pctx, rec(1)), 2.0 * T * nq * d)
        flop("prefill_attention", time_records(engine, pctx, rec(2)), 2.0 * T * T * dh * nh)
        flop("prefill_o", time_records(engine, pctx, rec(3)), 2.0 * T * d * nh * dh)
        flop("prefill_gate_up", time_records(engine, pctx, rec(5)), 2.0 * T * 2 * di * d)
        flop("prefill_down", time_records(engine, pctx, rec(6)), 2.0 * T * d * di)
        engine.end("kp")

    # ---- the plain path: one call per operator, library products, plain attention, norm kernels, no graphs ------
    plain = None
    vs_baseline = None
    if not args.no_plain:
        rt = engine.runtime
        saved = (rt.library_products_only, rt.plain_attention, rt.fused_norms, engine.runner.one_by_one, engine.use_graphs)
        rt.library_products_only, rt.plain_attention, rt.fused_norms = True, True, False
        engine.runner.one_by_one, engine.use_graphs = True, False
        plain = {"what": "one call per operator, library products, row attention kernel, norm kernels, no CUDA graphs"}
        for b in (1, 8, 64) if not args.no_points else (args.batch,):
            pm, _, _ = decode_device(b, args.context, 6, 3)
            plain[f"decode_b{b}"] = round(b * 1000.0 / pm, 1)
        if not args.no_prefill:
            T = 2048
            ptoks = torch.randint(0, V, (T,), generator=gen).tolist()
            times = []
            for i in range(3):
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                engine.step([StepEntry(f"pp{i}", ptoks, [T - 1])])
                e1.record()
                torch.cuda.synchronize()
                engine.end(f"pp{i}")
                if i >= 1:
                    times.append(e0.elapsed_time(e1))
            plain["prefill_ms"] = round(min(times), 3)
            plain["prefill_tok_s"] = round(T * 1000.0 / min(times), 1)
        (rt.library_products_only, rt.plain_attention, rt.fused_norms, engine.runner.one_by_one, engine.use_graphs) = saved
        base = plain.get(f"decode_b{args.batch}")
        vs_baseline = round(value / base, 3) if base else None

    meta_bytes = 4 * (7 * args.batch + 8 + args.batch * engine.cache.max_blocks * len(engine.cache.groups))
    line = {
        "metric": f"decode tok/s @ batch {args.batch} ({shape_name}, context {args.context})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": vs_baseline,
        "dtype": "bf16", "data": "synthetic: random-init weights N(0,0.02), uniform random token ids, random cache contents",
        "config": {
            "model": shape_name, "layers": cfg.num_hidden_layers, "layers_of_shape": full_layers,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "tied_embeddings": bool(cfg.tie_word_embeddings), "global_batch": args.batch, "seq_len": args.context,
            "context_len": args.context, "page_size": page, "parallelism": "single GPU",
            "l2": "inputs larger than L2: 5.4 GB of weights and the cache are re-read every step",
            "weights_gb": round(weight_bytes / 1e9, 3), "kv_bytes_per_token": kv_bytes_per_token,
        },
        "e2e": {"value": round(args.batch * 1000.0 / e2e_ms, 1), "unit": "tokens/s",
                "ms_per_step": round(e2e_ms, 4), "h2d_bytes_per_step": meta_bytes, "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": peak_source,
                     "bytes_per_step": int(step_bytes)},
        "clocks": clock_summary,
        "load_s": round(t_load, 1),
    }
    if prefill is not None:
        line["prefill"] = prefill
    if result_points:
        line["points"] = result_points
    if plain is not None:
        line["plain"] = plain
        line["baseline"] = "the engine's own plain path (the reference cannot be built here and publishes no number)"
    if kernel_block is not None:
        line["kernels"] = kernel_block
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
