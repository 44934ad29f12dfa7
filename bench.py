#!/usr/bin/env python3
"""Benchmark of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--workloads all|headline|14b|4b|rimopel|nagavik|fifudra|mefupel] [--impl reference]

Headline: decode tokens/s of the Qwen3-8B layer sizes (the baseline's third configuration) at batch 8 and context
4,096, the median of K device-timed steps after W warm-up steps; beside it batch 1 and 64, batch 8 at context 2,176
(a 2,048-token prompt half-way through 256 decoded tokens), batch 8 launched kernel by kernel instead of from a
captured graph, the prefill of one 2,048-token prompt, and the same decode loop end to end through ``LLM.step()``
(host token lists in, host tokens out).  Each with its fraction of the measured roofline.

Two more workloads run after it unless ``--workloads headline`` is given, both through ``LLM.step()`` and the scheduler:
* Qwen3-14B layer sizes, 8 prompts of 8,192 tokens fed in portions of 2,048, then 256 greedy tokens each;
* Qwen3-4B layer sizes, 32 requests with prompts of 128 to 4,096 tokens (seed 5) under a step budget of 2,048
  tokens, 128 new tokens each: prompt portions beside decoding.

Random weights drawn on the device, synthetic token ids.  One "step" is one decode step of the whole batch.  The
weights (8 to 28 GB) are far larger than L2, so no flush is needed between timed iterations.
"""
import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL_8B = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=40960,
                rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
MODEL_14B = dict(MODEL_8B, hidden_size=5120, intermediate_size=17408, num_hidden_layers=40, num_attention_heads=40)
MODEL_4B = dict(MODEL_8B, hidden_size=2560, intermediate_size=9728, tie_word_embeddings=True)
CONTEXT = 4096
WORKLOAD_CONTEXT = 2176     # a 2,048-token prompt half-way through its 256 decoded tokens
PREFILL_TOKENS = 2048
PAGE = 16


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples the SM clock and the throttle reasons of the GPU that the benchmark runs on (asked for by UUID:
    nvidia-smi's own indices ignore CUDA_VISIBLE_DEVICES) while the timed regions run.  Read-only."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu_id: str = "0"):
        self.rows, self.proc, self.gpu_id = [], None, gpu_id

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.gpu_id, f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def mark(self):
        return time.time()

    def stop(self):
        if self.proc:
            self.proc.terminate()

    def summary(self, windows):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, r in self.rows:
            if not any(a <= t <= (b or t) for a, b in windows) or len(r) < 6:
                continue
            try:
                sm.append(float(r[0])); mx = max(mx, float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm), "gpu": self.gpu_id}


def gpu_id_for_nvidia_smi(torch) -> str:
    """'GPU-<uuid>' of the CUDA device in use if nvidia-smi knows it under that name, else index 0."""
    try:
        uuid = str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
        name = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        r = subprocess.run(["nvidia-smi", "-i", name, "--query-gpu=uuid", "--format=csv,noheader"],
                           capture_output=True, text=True, timeout=20)
        if r.returncode == 0 and r.stdout.strip():
            return name
    except Exception:
        pass
    return "0"


def model_numbers(cfg):
    H, I, nh, nkv, hd, L, V = (cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                               cfg.head_dim, cfg.num_hidden_layers, cfg.vocab_size)
    layer_params = (nh + 2 * nkv) * hd * H + H * nh * hd + 3 * I * H
    tables = 1 if cfg.tie_word_embeddings else 2
    # a decode step reads every layer matrix, the LM head and the norm gains once; of the embedding table only the
    # rows of its tokens (a tied table is the LM head, read whole)
    weight_bytes = 2 * (L * layer_params + V * H) + 2 * L * (2 * H + 2 * hd) + 2 * H
    return dict(layer_params=layer_params, weight_bytes=weight_bytes, kv_bytes_per_token=L * 2 * nkv * hd * 2,
                stored_bytes=2 * (L * layer_params + tables * V * H))


def prefill_flops(cfg, T, past=0):
    """Products over T tokens, the LM head on one row, causal attention of T queries over past + their own keys."""
    n = model_numbers(cfg)
    L, nh, hd = cfg.num_hidden_layers, cfg.num_attention_heads, cfg.head_dim
    return 2.0 * T * L * n["layer_params"] + 2.0 * cfg.vocab_size * cfg.hidden_size + L * 4.0 * nh * hd * (T * past + T * (T + 1) / 2)


def release(*objs):
    import torch
    gc.collect()
    torch.cuda.empty_cache()


# ------------------------------------------------------------------------------------------------ headline: 8B
def run_headline(args, pk, clocks, windows):
    import numpy as np
    import torch
    from vllm_cpp_b200 import EngineConfig, LLM, Qwen3Config, ops
    from vllm_cpp_b200.engine.step import StepEntry
    from vllm_cpp_b200.runtime import runtime
    from vllm_cpp_b200.sampling import Sampler, SamplingOptions

    cfg = Qwen3Config(**dict(MODEL_8B, num_hidden_layers=args.layers))
    nums = model_numbers(cfg)
    points = [args.batch] if args.skip_points else sorted({1, args.batch, 64})
    max_seqs = max(points)
    # room for the end-to-end run, whose requests start decoding up to two steps apart each
    steps_total = args.steps + args.warmup + 2 * args.batch + 24
    per_req = -(-(args.context + steps_total) // 64) * 64
    max_tokens = max(max_seqs * per_req, 8192)
    t0 = time.time()
    llm = LLM(config=cfg, random_seed=0, engine=EngineConfig(dtype="bfloat16", page_size=PAGE, max_tokens=max_tokens,
                                                            max_num_seqs=max_seqs, max_step_tokens=PREFILL_TOKENS,
                                                            max_model_len=args.context + steps_total + 8,
                                                            cuda_graphs=not args.no_graphs))
    runner = llm.runner
    load_s = time.time() - t0
    rt = runtime()
    rng = np.random.default_rng(0)
    V = cfg.vocab_size
    GREEDY = SamplingOptions(0.0, 1.0, 1.0, 0)

    def fresh_cache():
        runner.reset_tables()
        return rt.CacheManager(runner.layout.runtime_groups(rt, PAGE, max_tokens // PAGE), max_seqs)

    # the cache of requests that "hold" a context: random keys and values stand for a processed prompt
    for t in runner.cache.tensors:
        for i in range(t.shape[0]):
            t[i].normal_(0, 1)

    def sample_post(ctx, logits):   # what LLM.step runs after the model, captured with the step
        return llm.sampler.sample_records(logits, ctx.user[:8 * logits.shape[0]].view(-1, 8), False, True)

    def decode_point(B, context, steps, warmup, graphs=True):
        runner.cuda_graphs = graphs and not args.no_graphs
        cm = fresh_cache()
        for r in range(B):
            cm.open(r)
            assert cm.reserve(r, context + steps + warmup + 1)
            cm.commit(r, context)
        times, launches = [], 0
        for it in range(warmup + steps):
            entries = []
            for r in range(B):
                pos = cm.num_tokens(r)
                entries.append(StepEntry(cm.slot(r), pos, [int(rng.integers(0, V))], [cm.block_table(r, 0)], [0]))
            if it == warmup:
                torch.cuda.synchronize()
                windows.append([clocks.mark(), None])
            l0 = ops.launch_count
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            flat, _, _ = Sampler.records([GREEDY] * B, [0] * B, [e.slot for e in entries])
            runner.step(entries, check=False, user=flat, post=sample_post, post_key=("sample", False, True))
            e1.record()
            e1.synchronize()
            if it >= warmup:
                times.append(e0.elapsed_time(e1))
                launches += ops.launch_count - l0
            for r in range(B):
                cm.commit(r, cm.num_tokens(r) + 1)
        windows[-1][1] = clocks.mark()
        ops.check_status(runner.status)
        runner.cuda_graphs = not args.no_graphs
        ms = statistics.median(times)
        nbytes = nums["weight_bytes"] + B * (context + warmup + steps / 2) * nums["kv_bytes_per_token"]
        gbs = nbytes / (ms * 1e-3) / 1e9
        return dict(ms=ms, mean_ms=sum(times) / len(times), tok_s=B * 1000.0 / ms, launches=launches, bytes=nbytes,
                    gbs=gbs, frac=gbs / pk["hbm_gbs"])

    results = {}
    if args.mode != "prefill":
        for B in points:
            results[("b", B)] = decode_point(B, args.context, args.steps, args.warmup)
        if not args.skip_points:
            results[("ctx", WORKLOAD_CONTEXT)] = decode_point(args.batch, WORKLOAD_CONTEXT, args.steps, args.warmup)
            results[("eager", args.batch)] = decode_point(args.batch, args.context, args.steps, args.warmup, graphs=False)
    if args.mode == "decode":
        print(json.dumps({"mode": "decode", "batch": args.batch, "context": args.context, "layers": args.layers,
                          "ms_per_step": {f"{k[0]}{k[1]}": v["ms"] for k, v in results.items()},
                          "roofline_frac": {f"{k[0]}{k[1]}": round(v["frac"], 4) for k, v in results.items()}}))
        return None
    head = results.get(("b", args.batch))

    # prefill: one prompt of 2,048 tokens in one step, logits of the last token only
    def prefill_once():
        cm = fresh_cache()
        cm.open(0)
        assert cm.reserve(0, PREFILL_TOKENS)
        ent = [StepEntry(cm.slot(0), 0, rng.integers(0, V, PREFILL_TOKENS).tolist(), [cm.block_table(0, 0)], [PREFILL_TOKENS - 1])]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step(ent, check=False)
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1)

    for _ in range(3):
        prefill_once()
    windows.append([clocks.mark(), None])
    pf = [prefill_once() for _ in range(9)]
    windows[-1][1] = clocks.mark()
    pf_ms = statistics.median(pf)
    T = PREFILL_TOKENS
    pf_flops = prefill_flops(cfg, T)
    if args.mode == "prefill":
        print(json.dumps({"mode": "prefill", "ms": pf_ms, "tokens_per_s": T * 1000.0 / pf_ms}))
        return None
    # frac: against the library's burst rate (one product timed alone); the back-to-back steps timed here run
    # under the power cap like the library's seconds-long loop, whose rate frac_of_sustained is taken against
    prefill = {"value": T * 1000.0 / pf_ms, "tokens": T, "ms": pf_ms, "frac": pf_flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12),
               "frac_of_sustained": pf_flops / (pf_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12)}

    # end to end through the Python entry point: host token lists in, host tokens out, every step
    B = args.batch
    e2e_steps = args.steps
    for r in range(B):
        llm.submit_tokens(rng.integers(0, V, args.context - args.warmup).tolist(), args.warmup + e2e_steps + 2 * B + 8, 0.0, 1.0,
                          repeat_penalty=1.0, ignore_eos=True)
    while True:   # feed the prompts; stop when every request is decoding
        o = llm.step()
        if len(o.new_token_ids) == B:
            break
    for _ in range(args.warmup - 1):
        llm.step()
    torch.cuda.synchronize()
    h0, d0 = llm.h2d_bytes, llm.d2h_bytes
    windows.append([clocks.mark(), None])
    step_s, n_tok = [], 0
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        t1 = time.perf_counter()
        n_tok += len(llm.step().new_token_ids)     # returns host tokens: the step has run when it comes back
        step_s.append(time.perf_counter() - t1)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    windows[-1][1] = clocks.mark()
    e2e_ms = 1000 * statistics.median(step_s)
    e2e = {"value": B * 1000.0 / e2e_ms, "unit": "tokens/s", "h2d_bytes_per_step": (llm.h2d_bytes - h0) / e2e_steps,
           "d2h_bytes_per_step": (llm.d2h_bytes - d0) / e2e_steps, "ms_per_step": e2e_ms,
           "mean_tokens_per_s": n_tok / e2e_s}

    name = {("b", 1): "decode_b1", ("b", 64): "decode_b64", ("ctx", WORKLOAD_CONTEXT): f"decode_b{args.batch}_ctx{WORKLOAD_CONTEXT}",
            ("eager", args.batch): f"decode_b{args.batch}_kernel_by_kernel"}
    line = {
        "metric": "decode tokens/s, Qwen3-8B shape, batch %d, context %d" % (args.batch, args.context),
        "value": head["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": head["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), uniform random token ids, random cache contents for the held context)",
        "impl": "ours",
        "config": {"model": "Qwen3-8B shape", "layers": cfg.num_hidden_layers, "layers_of_named_config": MODEL_8B["num_hidden_layers"],
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": V,
                   "global_batch": args.batch, "seq_len": args.context, "page_size": PAGE, "parallelism": "single GPU",
                   "l2": "inputs (16 GB of weights) larger than L2", "peaks": pk["source"], "timing": "median of steps, CUDA events"},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": head["gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": head["frac"]},
        "points": {name[k]: v["tok_s"] for k, v in results.items() if k in name},
        "points_ms": {name[k]: v["ms"] for k, v in results.items() if k in name},
        "points_roofline_frac": {name[k]: v["frac"] for k, v in results.items() if k in name},
        "mean_ms_per_step": head["mean_ms"],
        "e2e": e2e,
        "gpu_launches": head["launches"],
        "workspace_mb": runner.workspace.bytes() / 2 ** 20,
        "load_s": load_s,
    }
    del llm, runner
    release()
    return line


# ------------------------------------------------------------------------------------------------ 14B: long prompts, then decode
class GcPauses:
    """Seconds the Python collector ran inside a timed region (its pauses are the host's, so they belong to the
    end-to-end numbers; reported so that a slow run can be told from a slow engine)."""

    def __enter__(self):
        import gc
        self.total, self.count, self._t = 0.0, 0, 0.0
        gc.callbacks.append(self._cb)
        return self

    def _cb(self, phase, info):
        if phase == "start":
            self._t = time.perf_counter()
        else:
            self.total += time.perf_counter() - self._t
            self.count += 1

    def __exit__(self, *exc):
        import gc
        gc.callbacks.remove(self._cb)


def run_14b(args, pk, clocks, windows):
    """8 prompts of 8,192 tokens in portions of 2,048, then 256 greedy tokens each, through LLM.step()."""
    import numpy as np
    import torch
    from vllm_cpp_b200 import EngineConfig, LLM, Qwen3Config
    layers = args.layers_14b
    cfg = Qwen3Config(**dict(MODEL_14B, num_hidden_layers=layers))
    nums = model_numbers(cfg)
    B, P, NEW = 8, 8192, 256
    rng = np.random.default_rng(6)
    prompts = [rng.integers(0, cfg.vocab_size, P).tolist() for _ in range(B)]
    llm = LLM(config=cfg, random_seed=0, engine=EngineConfig(dtype="bfloat16", page_size=PAGE, max_tokens=B * (P + 320),
                                                            max_num_seqs=B, max_step_tokens=2048, max_model_len=P + 320))
    llm.warm_up(0.0, 1.0, 1.0)       # the captured decoding steps are made before the clock starts, as at a server's start
    for p in prompts:
        llm.submit_tokens(p, NEW, 0.0, 1.0, repeat_penalty=1.0, ignore_eos=True)
    torch.cuda.synchronize()
    windows.append([clocks.mark(), None])
    t0 = time.perf_counter()
    prefill_steps, decode_s, first_decode = 0, [], None
    flops = 0.0
    with GcPauses() as pauses:
        while llm.has_requests():
            t1 = time.perf_counter()
            o = llm.step()
            dt = time.perf_counter() - t1
            if o.num_prompt_tokens:
                prefill_steps += 1
            else:
                if first_decode is None:
                    torch.cuda.synchronize()
                    first_decode = t1
                decode_s.append(dt)
        torch.cuda.synchronize()
    windows[-1][1] = clocks.mark()
    prefill_s = first_decode - t0
    for _ in range(B):     # each prompt: four portions of 2,048 over what came before
        flops += sum(prefill_flops(cfg, 2048, past) for past in range(0, P, 2048))
    ms = 1000 * statistics.median(decode_s)
    nbytes = nums["weight_bytes"] + B * (P + NEW / 2) * nums["kv_bytes_per_token"]
    out = {"model": "Qwen3-14B shape", "layers": layers, "layers_of_named_config": MODEL_14B["num_hidden_layers"],
           "requests": B, "prompt_tokens_each": P, "portion": 2048, "new_tokens_each": NEW,
           "prefill_tokens_per_s": B * P / prefill_s, "prefill_s": prefill_s, "prefill_steps": prefill_steps,
           "prefill_frac_of_sustained": flops / prefill_s / (pk["bf16_tflops_sustained"] * 1e12),
           "decode_tokens_per_s": B * 1000.0 / ms, "decode_ms_per_step": ms, "decode_steps": len(decode_s),
           "decode_roofline_frac": nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"],
           "preemptions": llm.stats().preemptions, "python_gc_s": round(pauses.total, 4), "python_gc_runs": pauses.count,
           "through": "LLM.step() and the scheduler, host tokens in and out"}
    del llm
    release()
    return out


# ------------------------------------------------------------------------------------------------ 4B: a mixed batch
def run_4b(args, pk, clocks, windows):
    """32 requests, prompts of 128 to 4,096 tokens (seed 5), step budget 2,048 tokens, 128 new tokens each."""
    import numpy as np
    import torch
    from vllm_cpp_b200 import EngineConfig, LLM, Qwen3Config
    layers = args.layers_4b
    cfg = Qwen3Config(**dict(MODEL_4B, num_hidden_layers=layers))
    rng = np.random.default_rng(5)
    lens = rng.integers(128, 4097, 32).tolist()
    prompts = [rng.integers(0, cfg.vocab_size, n).tolist() for n in lens]
    total = sum(lens)
    NEW = 128
    max_tokens = -(-(total + 32 * (NEW + 64)) // 64) * 64
    llm = LLM(config=cfg, random_seed=0, engine=EngineConfig(dtype="bfloat16", page_size=PAGE, max_tokens=max_tokens,
                                                            max_num_seqs=32, max_step_tokens=2048, max_model_len=4096 + NEW + 128))
    warmed = llm.warm_up(0.0, 1.0, 1.0)       # the captured decoding steps are made before the clock starts, as at a server's start
    for p in prompts:
        llm.submit_tokens(p, NEW, 0.0, 1.0, repeat_penalty=1.0, ignore_eos=True)
    cache = llm.scheduler.cache()
    torch.cuda.synchronize()
    windows.append([clocks.mark(), None])
    t0 = time.perf_counter()
    steps = gen = mixed_steps = 0
    fewest_free = cache.free_pages(0)
    while llm.has_requests():
        o = llm.step()
        fewest_free = min(fewest_free, cache.free_pages(0))     # read after each step: the pool's high-water mark
        steps += 1
        gen += len(o.new_token_ids)
        mixed_steps += bool(o.num_prompt_tokens and o.num_generation_tokens)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    windows[-1][1] = clocks.mark()
    st = llm.stats()
    out = {"model": "Qwen3-4B shape", "layers": layers, "layers_of_named_config": MODEL_4B["num_hidden_layers"],
           "requests": 32, "prompt_tokens": total, "new_tokens_each": NEW, "step_token_budget": 2048,
           "total_tokens_per_s": (total + gen) / dt, "generated_tokens_per_s": gen / dt, "seconds": dt, "steps": steps,
           "steps_with_portions_beside_decoding": mixed_steps, "mean_step_ms": 1000 * dt / steps,
           "pages_high_water": max_tokens // PAGE - fewest_free, "pages_in_pool": max_tokens // PAGE, "preemptions": st.preemptions,
           "graph_replays": llm.runner.graph_replays, "decoding_steps_captured_before_the_clock": warmed,
           "through": "LLM.step() and the scheduler, host tokens in and out"}
    del llm
    release()
    return out


# ------------------------------------------------------------------------------------------------ Rimopel beside Qwen3
# Layer sizes of real models (random weights): width, heads, KV heads, head size, the dense feed-forward's hidden size and
# the SwiGLU hidden size with as many parameters, window, layers.
RIMOPEL_SIZES = {
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, swiglu=5504, window=1024, layers=12, vocab=32768),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=16384, swiglu=10944, window=2048, layers=8, vocab=32768),
}


def run_beside(args, pk, clocks, windows, workload, sizes, configs, numbers):
    """Prefill (one prompt of 2,048 tokens in one step) and decode (a batch behind a context of 4,096 tokens, captured
    steps) of a design at real layer sizes beside Qwen3 at equal size: tokens/s, the fraction of the measured roofline
    (each model's own work counted), and the time per group of kernels.  ``configs(z)``: name -> configuration;
    ``numbers(z, name)``: weight_bytes and per-request cache_bytes a decode step reads, and the prefill's flops."""
    import numpy as np
    import torch
    from vllm_cpp_b200 import EngineConfig, LLM, ops
    from vllm_cpp_b200.engine.step import StepEntry
    from vllm_cpp_b200.runtime import runtime

    rt = runtime()
    rng = np.random.default_rng(0)
    B, context, T = args.batch, args.context, PREFILL_TOKENS
    out = {"workload": workload, "batch": B, "context": context, "prefill_tokens": T, "peaks": pk["source"],
           "data": "synthetic (random weights, uniform random token ids, random cache contents for the held context)",
           "l2": "inputs (over 1 GB of weights) larger than L2", "timing": "median of steps, CUDA events", "sizes": {}}

    def measure(cfg, z, name, profile):
        per_req = -(-(context + args.steps + args.warmup + 8) // 64) * 64
        max_tokens = max(B * per_req, T + 64)
        llm = LLM(config=cfg, random_seed=0, engine=EngineConfig(dtype="bfloat16", page_size=PAGE, max_tokens=max_tokens, max_num_seqs=B,
                                                                max_step_tokens=T, max_model_len=context + 4096, profile=profile))
        runner = llm.runner
        V = z["vocab"]
        for g, t in zip(runner.layout.groups, runner.cache.tensors):
            for i in range(t.shape[0]):
                t[i].normal_(0, 1 if g.paged else 0.01)
        n_groups = len(runner.layout.paged)

        def fresh():
            runner.reset_tables()
            return rt.CacheManager(runner.layout.runtime_groups(rt, PAGE, max_tokens // PAGE), B)

        def timed(fn, n, warm):
            times = []
            for it in range(warm + n):
                if it == warm:
                    windows.append([clocks.mark(), None])
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ent = fn()
                e0.record()
                runner.step(ent, check=False)
                e1.record()
                e1.synchronize()
                times.append(e0.elapsed_time(e1))
            windows[-1][1] = clocks.mark()
            return statistics.median(times[warm:])

        def prefill_entry():
            cm = fresh()
            cm.open(0)
            assert cm.reserve(0, T)
            return [StepEntry(cm.slot(0), 0, rng.integers(0, V, T).tolist(), [cm.block_table(0, g) for g in range(n_groups)], [T - 1])]

        res = {}
        if profile:
            runner.profile.clear()
        l0 = ops.launch_count
        pf_ms = timed(prefill_entry, 5, 3)
        res["prefill_launches"] = (ops.launch_count - l0) // 8
        if profile:
            res["prefill_groups_ms"] = {k: round(v / 8, 4) for k, v in sorted(runner.profile.items())}
            runner.profile.clear()
        cm = fresh()
        for r in range(B):
            cm.open(r)
            assert cm.reserve(r, context + args.steps + args.warmup + 1)
            cm.commit(r, context)

        def decode_entries():
            ent = []
            for r in range(B):
                pos = cm.num_tokens(r)
                ent.append(StepEntry(cm.slot(r), pos, [int(rng.integers(0, V))], [cm.block_table(r, g) for g in range(n_groups)], [0]))
                cm.commit(r, pos + 1)
            return ent

        dec_ms = timed(decode_entries, args.steps, args.warmup)
        if profile:
            res["decode_groups_ms"] = {k: round(v / (args.steps + args.warmup), 4) for k, v in sorted(runner.profile.items())}
        ops.check_status(runner.status)
        n = numbers(z, name)
        res.update(prefill_ms=pf_ms, prefill_tokens_per_s=T * 1000.0 / pf_ms,
                   prefill_frac_of_bf16_peak=n["prefill_flops"] / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12),
                   decode_ms=dec_ms, decode_tokens_per_s=B * 1000.0 / dec_ms,
                   decode_frac_of_hbm_peak=(n["weight_bytes"] + B * n["cache_bytes"]) / (dec_ms * 1e-3) / 1e9 / pk["hbm_gbs"])
        del llm, runner
        release()
        return res

    for size, z in sizes.items():
        if args.size and size != args.size:
            continue
        out["sizes"][size] = {"config": z}
        for name, cfg in configs(z).items():
            r = measure(cfg, z, name, profile=False)
            p = measure(cfg, z, name, profile=True)      # kernel by kernel, with events between the groups of kernels
            r["prefill_groups_ms"], r["decode_groups_ms"] = p["prefill_groups_ms"], p["decode_groups_ms"]
            r["prefill_launches"] = p["prefill_launches"]
            out["sizes"][size][name] = r
    return out


def run_rimopel(args, pk, clocks, windows):
    """Rimopel at real layer sizes beside Qwen3 with the same width, heads, window on every layer, layer count and
    feed-forward parameter count (see run_beside)."""
    from vllm_cpp_b200 import Qwen3Config
    from vllm_cpp_b200.config.rimopel import RimopelConfig, RimopelLayer, RimopelMixer
    context, T = args.context, PREFILL_TOKENS

    def configs(z):
        mixer = RimopelMixer(heads=z["heads"], kv_heads=z["kv_heads"], dim=z["dim"], vdim=z["dim"], scale=z["dim"] ** -0.5, conv=3,
                             window=z["window"], keep_first=4)
        rim = RimopelConfig(vocab=z["vocab"], width=z["width"], norm_eps=1e-5, canon_taps=3, max_positions=context + 4096,
                            layers=tuple(RimopelLayer("attention", mixer, "dense", z["ff"]) for _ in range(z["layers"])))
        qwen = Qwen3Config(vocab_size=z["vocab"], hidden_size=z["width"], intermediate_size=z["swiglu"], num_hidden_layers=z["layers"],
                           num_attention_heads=z["heads"], num_key_value_heads=z["kv_heads"], head_dim=z["dim"],
                           max_position_embeddings=context + 4096, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False,
                           sliding_window=z["window"], layer_types=("sliding_attention",) * z["layers"])
        return {"rimopel": rim, "qwen3": qwen}

    def numbers(z, name):
        W, H, G, d, L, V = z["width"], z["heads"], z["kv_heads"], z["dim"], z["layers"], z["vocab"]
        attn = (H + 2 * G) * d * W + W * H * d
        layer = attn + (2 * z["ff"] * W + 2 * W * W if name == "rimopel" else 3 * z["swiglu"] * W)
        keys = min(context, z["window"])
        return dict(weight_bytes=2 * (L * layer + V * W), cache_bytes=L * 2 * G * d * 2 * keys,
                    prefill_flops=2.0 * T * L * layer + 2.0 * V * W + L * 4.0 * H * d * sum(min(i + 1, z["window"]) for i in range(T)))

    return run_beside(args, pk, clocks, windows, "rimopel_beside_qwen3", RIMOPEL_SIZES, configs, numbers)


# Nagavik at real layer sizes: two recurrent layers, then one attention layer, and so on; every layer with routed experts
# (two of sixteen) and a shared expert.  Qwen3 beside it has the same width, heads, layer count (attention on every
# layer) and as many feed-forward parameters per token as Nagavik has active ones (three matrices of width x ff).
NAGAVIK_SIZES = {
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, ssm_heads=64, ssm_vdim=64, state=128, groups=8, experts=16, top=2,
                  ff=2048, shared=2048, swiglu=4096, layers=12, vocab=32768),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, ssm_heads=128, ssm_vdim=64, state=128, groups=8, experts=16, top=2,
                  ff=4096, shared=4096, swiglu=8192, layers=8, vocab=32768),
}


def nagavik_kinds(z):
    return ["attention" if i % 3 == 2 else "mamba2" for i in range(z["layers"])]


def nagavik_config(z, context):
    from vllm_cpp_b200.config.nagavik import NagavikAttention, NagavikConfig, NagavikLayer, NagavikMamba2, NagavikMlp
    attn = NagavikAttention(heads=z["heads"], kv_heads=z["kv_heads"], dim=z["dim"], vdim=z["dim"], scale=z["dim"] ** -0.5, softcap=50.0)
    ssm = NagavikMamba2(heads=z["ssm_heads"], vdim=z["ssm_vdim"], state=z["state"], groups=z["groups"], conv=4, norm_groups=z["groups"])
    mlp = NagavikMlp("moe", ff=z["ff"], experts=z["experts"], top=z["top"], shared_ff=z["shared"])
    return NagavikConfig(vocab=z["vocab"], width=z["width"], max_positions=context + 4096, norm_eps=1e-5, embedding_scale=1.0,
                         logit_softcap=30.0,
                         layers=tuple(NagavikLayer(k, attn if k == "attention" else ssm, mlp) for k in nagavik_kinds(z)))


def nagavik_numbers(z, context, T, B):
    W, H, G, d, L, V = z["width"], z["heads"], z["kv_heads"], z["dim"], z["layers"], z["vocab"]
    attn_w = (H + 2 * G) * d * W + W * H * d
    attn_flops = 4.0 * H * d * sum(i + 1 for i in range(T))
    n_attn = nagavik_kinds(z).count("attention")
    n_ssm = L - n_attn
    inner, gn = z["ssm_heads"] * z["ssm_vdim"], z["groups"] * z["state"]
    ssm_w = (2 * inner + 2 * gn + z["ssm_heads"]) * W + W * inner
    expert = 2 * z["ff"] * W
    ff_active = z["top"] * expert + 2 * z["shared"] * W + z["experts"] * W
    # experts a decode step reads: the distinct ones B tokens choose, in expectation
    distinct = z["experts"] * (1.0 - (1.0 - z["top"] / z["experts"]) ** B)
    ff_read = distinct * expert + 2 * z["shared"] * W + z["experts"] * W
    state_bytes = 2 * 4 * inner * z["state"]       # read and written, 32-bit
    return dict(weight_bytes=2 * (n_attn * attn_w + n_ssm * ssm_w + L * ff_read + V * W),
                cache_bytes=n_attn * 2 * G * d * 2 * context + n_ssm * state_bytes,
                prefill_flops=2.0 * T * (n_attn * attn_w + n_ssm * ssm_w + L * ff_active) + 2.0 * V * W + n_attn * attn_flops
                              + n_ssm * 6.0 * T * inner * z["state"])


def run_nagavik(args, pk, clocks, windows):
    """Nagavik at real layer sizes beside Qwen3 at equal size (see NAGAVIK_SIZES and run_beside)."""
    from vllm_cpp_b200 import Qwen3Config
    context, T, B = args.context, PREFILL_TOKENS, args.batch

    def configs(z):
        qwen = Qwen3Config(vocab_size=z["vocab"], hidden_size=z["width"], intermediate_size=z["swiglu"], num_hidden_layers=z["layers"],
                           num_attention_heads=z["heads"], num_key_value_heads=z["kv_heads"], head_dim=z["dim"],
                           max_position_embeddings=context + 4096, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
        return {"nagavik": nagavik_config(z, context), "qwen3": qwen}

    def numbers(z, name):
        W, H, G, d, L, V = z["width"], z["heads"], z["kv_heads"], z["dim"], z["layers"], z["vocab"]
        if name == "qwen3":
            attn_w = (H + 2 * G) * d * W + W * H * d
            layer = attn_w + 3 * z["swiglu"] * W
            return dict(weight_bytes=2 * (L * layer + V * W), cache_bytes=L * 2 * G * d * 2 * context,
                        prefill_flops=2.0 * T * L * layer + 2.0 * V * W + L * 4.0 * H * d * sum(i + 1 for i in range(T)))
        return nagavik_numbers(z, context, T, B)

    return run_beside(args, pk, clocks, windows, "nagavik_beside_qwen3", NAGAVIK_SIZES, configs, numbers)


# Fifudra at real layer sizes beside Nagavik, the closest design the engine has (recurrent layers with an attention layer
# after every two, routed experts on every layer), at equal width, layer count, recurrent state per request and active
# feed-forward parameters per token: a delta-rule layer, a gated linear layer, an attention layer through a latent, and so
# on; four residual streams; four of sixteen gated experts chosen within two of four groups.
FIFUDRA_SIZES = {
    "w2048": dict(NAGAVIK_SIZES["w2048"], f_heads=16, f_dim=128, f_rot=32, f_vdim=128, q_rank=768, kv_rank=96, r_heads=16, r_kv_heads=8,
                  r_dim=128, r_vdim=256, f_ff=1024, f_top=4, f_groups=4, f_keep=2, streams=4),
    "w4096": dict(NAGAVIK_SIZES["w4096"], f_heads=32, f_dim=128, f_rot=32, f_vdim=128, q_rank=1536, kv_rank=96, r_heads=32, r_kv_heads=16,
                  r_dim=128, r_vdim=256, f_ff=2048, f_top=4, f_groups=4, f_keep=2, streams=4),
    # cached rows of 256 lanes: wider than the attention kernels on the tensor cores take (the plain kernel runs)
    "w2048_k256": dict(NAGAVIK_SIZES["w2048"], f_heads=16, f_dim=128, f_rot=64, f_vdim=128, q_rank=768, kv_rank=192, r_heads=16,
                       r_kv_heads=8, r_dim=128, r_vdim=256, f_ff=1024, f_top=4, f_groups=4, f_keep=2, streams=4),
}


def run_fifudra(args, pk, clocks, windows):
    """Fifudra at real layer sizes beside Nagavik at equal size (see FIFUDRA_SIZES and run_beside)."""
    from vllm_cpp_b200.config.fifudra import (DeltaSpec, FifudraConfig, FifudraLayer, FifudraMlp, Hgrn2Spec, LatentAttentionSpec,
                                              RotarySpec)
    context, T, B = args.context, PREFILL_TOKENS, args.batch

    def kinds(z):
        return [("delta", "hgrn2", "latent_attention")[i % 3] for i in range(z["layers"])]

    def configs(z):
        mixers = {"delta": DeltaSpec(heads=z["r_heads"], kv_heads=z["r_kv_heads"], dim=z["r_dim"], vdim=z["r_vdim"], conv=4),
                  "hgrn2": Hgrn2Spec(heads=z["r_heads"], dim=z["r_dim"], vdim=z["r_vdim"]),
                  "latent_attention": LatentAttentionSpec(
                      heads=z["f_heads"], dim=z["f_dim"], rot_dim=z["f_rot"], vdim=z["f_vdim"], q_rank=z["q_rank"], kv_rank=z["kv_rank"],
                      scale=(z["f_dim"] + z["f_rot"]) ** -0.5,
                      rot=RotarySpec(base=1e6, dims=z["f_rot"], factor=4.0, original=4096.0, fast=32.0, slow=1.0))}
        mlp = FifudraMlp("moe", ff=z["f_ff"], experts=z["experts"], top=z["f_top"], scale=1.0, groups=z["f_groups"], keep=z["f_keep"])
        fif = FifudraConfig(vocab=z["vocab"], width=z["width"], norm_eps=1e-5, embedding_scale=1.0, streams=z["streams"],
                            max_positions=context + 4096, layers=tuple(FifudraLayer(k, mixers[k], mlp) for k in kinds(z)))
        return {"fifudra": fif, "nagavik": nagavik_config(z, context)}

    def numbers(z, name):
        if name == "nagavik":
            return nagavik_numbers(z, context, T, B)
        W, L, V = z["width"], z["layers"], z["vocab"]
        H, d, r, vd, qr, kr = z["f_heads"], z["f_dim"], z["f_rot"], z["f_vdim"], z["q_rank"], z["kv_rank"]
        RH, RG, rd, rv = z["r_heads"], z["r_kv_heads"], z["r_dim"], z["r_vdim"]
        n = {k: kinds(z).count(k) for k in ("delta", "hgrn2", "latent_attention")}
        lat_w = (qr + kr + r) * W + H * (d + r) * qr + H * d * kr + H * vd * kr + W * H * vd
        delta_w = (2 * RG * rd + 2 * RH * rv + 2 * RH) * W + W * RH * rv
        hgrn_w = (2 * RH * rd + RH * rv) * W + W * RH * rv
        expert = 3 * z["f_ff"] * W
        ff_active = z["f_top"] * expert + z["experts"] * W
        distinct = z["experts"] * (1.0 - (1.0 - z["f_top"] / z["experts"]) ** B)
        ff_read = distinct * expert + z["experts"] * W
        mixers_w = n["latent_attention"] * lat_w + n["delta"] * delta_w + n["hgrn2"] * hgrn_w
        state_bytes = 2 * 4 * RH * rd * rv              # read and written, 32-bit
        keys = sum(i + 1 for i in range(T))
        return dict(weight_bytes=2 * (mixers_w + L * ff_read + V * W),
                    # a cached token: the key row [latent | rotated part] and the value row (the latent), 16-bit
                    cache_bytes=n["latent_attention"] * (2 * kr + r) * 2 * context + (n["delta"] + n["hgrn2"]) * state_bytes,
                    prefill_flops=2.0 * T * (mixers_w + L * ff_active) + 2.0 * V * W
                                  + n["latent_attention"] * 2.0 * H * (2 * kr + r) * keys
                                  + (6.0 * n["delta"] + 4.0 * n["hgrn2"]) * T * RH * rd * rv)

    return run_beside(args, pk, clocks, windows, "fifudra_beside_nagavik", FIFUDRA_SIZES, configs, numbers)


# Mefupel at real layer sizes beside Fifudra, the closest design the engine has (recurrences on a matrix state per head
# between attention layers, a stretch of layers that runs twice), at equal width, layer count, repeated stretch,
# recurrent state per request and feed-forward parameters: a gated-linear-attention layer, a layer of window attention
# beside retention, a window attention layer with turned values, and so on, each with a dense feed-forward of two
# matrices; Fifudra with its dense gated feed-forward of three.
MEFUPEL_SIZES = {
    "w2048": dict(width=2048, layers=12, loop=(3, 6, 2), vocab=32768, heads=16, kv_heads=4, dim=128, window=1024, rot=64,
                  r_heads=16, r_dim=128, r_vdim=256, rank=64, ff=6144,
                  f_heads=16, f_dim=128, f_rot=32, f_vdim=128, q_rank=768, kv_rank=96, r_kv_heads=8, f_ff=4096, streams=4),
    "w4096": dict(width=4096, layers=8, loop=(2, 5, 2), vocab=32768, heads=32, kv_heads=8, dim=128, window=2048, rot=64,
                  r_heads=32, r_dim=128, r_vdim=256, rank=128, ff=12288,
                  f_heads=32, f_dim=128, f_rot=32, f_vdim=128, q_rank=1536, kv_rank=96, r_kv_heads=16, f_ff=8192, streams=4),
}


def run_mefupel(args, pk, clocks, windows):
    """Mefupel at real layer sizes beside Fifudra at equal size (see MEFUPEL_SIZES and run_beside)."""
    from vllm_cpp_b200.config.fifudra import (DeltaSpec, FifudraConfig, FifudraLayer, FifudraMlp, Hgrn2Spec, LatentAttentionSpec,
                                              RotarySpec)
    from vllm_cpp_b200.config.mefupel import (AttentionSpec, GlaSpec, MefupelConfig, MefupelLayer, MefupelMlp, ParallelSpec,
                                              RetentionSpec, Rotation)
    context, T = args.context, PREFILL_TOKENS

    def kinds(z):
        return [("gla", "parallel", "attention")[i % 3] for i in range(z["layers"])]

    def fifudra_kinds(z):
        return [("delta", "hgrn2", "latent_attention")[i % 3] for i in range(z["layers"])]

    def runs(z, names):
        a, b, n = z["loop"]
        return names[:a] + names[a:b] * n + names[b:]

    def configs(z):
        H, G, d, RH = z["heads"], z["kv_heads"], z["dim"], z["r_heads"]
        attn = AttentionSpec(heads=H, kv_heads=G, dim=d, vdim=d, scale=d ** -0.5, window=z["window"], rot=Rotation(1e6, d))
        left = AttentionSpec(heads=H, kv_heads=G, dim=d, vdim=d, scale=d ** -0.5, window=z["window"], rot=Rotation(5e5, z["rot"]))
        right = RetentionSpec(heads=RH, dim=z["r_dim"], vdim=z["r_vdim"], decay=tuple(1.0 - 2.0 ** (-5 - 6 * i / max(RH - 1, 1)) for i in range(RH)),
                              rot=Rotation(1e6, z["r_dim"]))
        mixers = {"gla": GlaSpec(heads=RH, dim=z["r_dim"], vdim=z["r_vdim"], tau=16.0, rank=z["rank"]), "parallel": ParallelSpec(left, right),
                  "attention": attn}
        a, b, n = z["loop"]
        mef = MefupelConfig(vocab=z["vocab"], width=z["width"], norm_eps=1e-5, has_loop=True, loop_start=a, loop_stop=b, loop_times=n,
                            max_positions=context + 4096,
                            layers=tuple(MefupelLayer(k, mixers[k], MefupelMlp("dense", z["ff"])) for k in kinds(z)))
        fmix = {"delta": DeltaSpec(heads=RH, kv_heads=z["r_kv_heads"], dim=z["r_dim"], vdim=z["r_vdim"], conv=4),
                "hgrn2": Hgrn2Spec(heads=RH, dim=z["r_dim"], vdim=z["r_vdim"]),
                "latent_attention": LatentAttentionSpec(
                    heads=z["f_heads"], dim=z["f_dim"], rot_dim=z["f_rot"], vdim=z["f_vdim"], q_rank=z["q_rank"], kv_rank=z["kv_rank"],
                    scale=(z["f_dim"] + z["f_rot"]) ** -0.5, rot=RotarySpec(base=1e6, dims=z["f_rot"]))}
        fif = FifudraConfig(vocab=z["vocab"], width=z["width"], norm_eps=1e-5, embedding_scale=1.0, streams=z["streams"],
                            loop_start=a, loop_stop=b, loop_times=n, max_positions=context + 4096,
                            layers=tuple(FifudraLayer(k, fmix[k], FifudraMlp("dense", ff=z["f_ff"])) for k in fifudra_kinds(z)))
        return {"mefupel": mef, "fifudra": fif}

    def numbers(z, name):
        W, V = z["width"], z["vocab"]
        RH, rd, rv = z["r_heads"], z["r_dim"], z["r_vdim"]
        state_bytes = 2 * 4 * RH * rd * rv              # read and written, 32-bit
        if name == "fifudra":
            H, d, r, vd, qr, kr, RG = z["f_heads"], z["f_dim"], z["f_rot"], z["f_vdim"], z["q_rank"], z["kv_rank"], z["r_kv_heads"]
            order = runs(z, fifudra_kinds(z))
            n = {k: order.count(k) for k in ("delta", "hgrn2", "latent_attention")}
            w = {"latent_attention": (qr + kr + r) * W + H * (d + r) * qr + H * d * kr + H * vd * kr + W * H * vd,
                 "delta": (2 * RG * rd + 2 * RH * rv + 2 * RH) * W + W * RH * rv, "hgrn2": (2 * RH * rd + RH * rv) * W + W * RH * rv}
            weights = sum(n[k] * w[k] for k in n) + len(order) * 3 * z["f_ff"] * W
            return dict(weight_bytes=2 * (weights + V * W),
                        cache_bytes=n["latent_attention"] * (2 * kr + r) * 2 * context + (n["delta"] + n["hgrn2"]) * state_bytes,
                        prefill_flops=2.0 * T * weights + 2.0 * V * W + n["latent_attention"] * 2.0 * H * (2 * kr + r) * sum(i + 1 for i in range(T))
                                      + (6.0 * n["delta"] + 4.0 * n["hgrn2"]) * T * RH * rd * rv)
        H, G, d = z["heads"], z["kv_heads"], z["dim"]
        order = runs(z, kinds(z))
        n = {k: order.count(k) for k in ("gla", "parallel", "attention")}
        attn_w = (H + 2 * G) * d * W + W * H * d
        left_w = (H + G) * d * W + W * H * d
        rec_w = (2 * RH * rd + 2 * RH * rv) * W + W * RH * rv
        w = {"attention": attn_w, "parallel": left_w + rec_w, "gla": rec_w + z["rank"] * (W + RH * rd)}
        weights = sum(n[k] * w[k] for k in n) + len(order) * 2 * z["ff"] * W
        keys = min(context, z["window"])
        seen = sum(min(i + 1, z["window"]) for i in range(T))
        return dict(weight_bytes=2 * (weights + V * W),
                    # a cached token: a key row and a value row per KV head, 16-bit
                    cache_bytes=(n["attention"] + n["parallel"]) * 2 * G * d * 2 * keys + (n["gla"] + n["parallel"]) * state_bytes,
                    prefill_flops=2.0 * T * weights + 2.0 * V * W + (n["attention"] + n["parallel"]) * 4.0 * H * d * seen
                                  + 4.0 * (n["gla"] + n["parallel"]) * T * RH * rd * rv)

    return run_beside(args, pk, clocks, windows, "mefupel_beside_fifudra", MEFUPEL_SIZES, configs, numbers)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--layers", type=int, default=MODEL_8B["num_hidden_layers"])
    ap.add_argument("--layers-14b", type=int, default=MODEL_14B["num_hidden_layers"])
    ap.add_argument("--layers-4b", type=int, default=MODEL_4B["num_hidden_layers"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workloads", default="all", choices=["all", "headline", "14b", "4b", "rimopel", "nagavik", "fifudra", "mefupel"],
                    help="headline: the 8B numbers only; 14b / 4b: that workload alone (prints its own JSON line); rimopel, "
                         "nagavik: that design at real layer sizes beside Qwen3 at equal size, prefill and decode (its own JSON line); "
                         "fifudra: that design beside Nagavik at equal size, likewise; mefupel: that design beside Fifudra at equal size, likewise")
    ap.add_argument("--size", default="", help="rimopel, nagavik, fifudra, mefupel: one of the workload's sizes only (w2048, w4096; fifudra also w2048_k256)")
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch (for profiling runs)")
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel (for profiling runs)")
    ap.add_argument("--mode", default="all", choices=["all", "decode", "prefill"], help="what to run (profiling runs)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "laik/vllm-cpp has no Python package or installable build (pip finds no setup.py/pyproject.toml), "
                          "its CUDA sources do not compile with nvcc 12.9, and its CUDA forward has attention stubbed out"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    pk = peaks()
    clocks = ClockSampler(gpu_id_for_nvidia_smi(torch))
    clocks.start()
    windows = []
    try:
        if args.workloads in ("14b", "4b", "rimopel", "nagavik", "fifudra", "mefupel"):
            out = {"14b": run_14b, "4b": run_4b, "rimopel": run_rimopel, "nagavik": run_nagavik, "fifudra": run_fifudra, "mefupel": run_mefupel}[args.workloads](args, pk, clocks, windows)
            out["clocks"] = clocks.summary(windows)
            print(json.dumps(out))
            return 0
        line = run_headline(args, pk, clocks, windows)
        if line is None:
            return 0
        line["clocks"] = clocks.summary(windows)      # of the 8B runs; the other workloads carry their own
        if args.workloads == "all" and args.mode == "all" and not args.skip_points:
            extra = {}
            for key, fn in (("qwen3_14b_long_prompts", run_14b), ("qwen3_4b_mixed_batch", run_4b)):
                w = []
                try:
                    extra[key] = fn(args, pk, clocks, w)
                    extra[key]["clocks"] = clocks.summary(w)
                except Exception as e:   # the headline stands even if a further workload cannot run (memory, time)
                    extra[key] = {"error": f"{type(e).__name__}: {e}"[:300]}
                    release()
            line["workloads"] = extra
        print(json.dumps(line))
        return 0
    finally:
        clocks.stop()


if __name__ == "__main__":
    sys.exit(main())
