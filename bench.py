#!/usr/bin/env python3
"""Decode and prefill throughput of mini_infer_b200 on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The model has the layer sizes of Qwen1.5-MoE-A2.7B (24 layers, hidden 2048, 16 heads of 128,
60 experts of 1408 with top-4 routing, a shared expert of 5632, vocabulary 151936), random
bfloat16 weights and seeded uniform-random token ids.  The headline ``value`` is decoded tokens
per second at batch 8 with 2,048-token prompts in a 4,096-token context: K timed decode steps,
timed on the device with CUDA events after W warm-up steps.  ``e2e`` is the same metric through
the Python entry point ``LLM.generate`` (host token ids in, host token ids out; every step stages its
inputs in pinned memory, copies them to the device and reads the sampled ids back): the wall time
of generating K+1 tokens per prompt minus that of generating 1, so that the prompts' prefill
cancels.  ``prefill`` times one 2,048-token prompt; ``points`` holds
decode at batch 1 and 64; ``roofline`` divides the bytes a decode step must read (every weight it
uses once, the cache of the live requests) by its time.  Every step reads far more than the
126 MB of L2 (gigabytes of weights), so no separate flush is needed between timed iterations.
"""

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the headline configuration: Qwen1.5-MoE-A2.7B layer sizes
A27B = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "vocab_size": 151936, "hidden_size": 2048, "intermediate_size": 5632, "num_hidden_layers": 24,
    "num_attention_heads": 16, "num_key_value_heads": 16, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "max_position_embeddings": 8192, "tie_word_embeddings": False, "hidden_act": "silu",
    "num_experts": 60, "num_experts_per_tok": 4, "moe_intermediate_size": 1408,
    "shared_expert_intermediate_size": 5632, "norm_topk_prob": False, "decoder_sparse_step": 1,
    "mlp_only_layers": [], "use_sliding_window": False, "sliding_window": 32768, "max_window_layers": 21,
}
FULL_LAYERS = 24
# Qwen2-57B-A14B layer sizes (the second bf16 configuration: decode at batch 1 and 8, 1,024-token prompts)
A14B = dict(A27B, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28, num_attention_heads=28,
            num_key_value_heads=4, num_experts=64, num_experts_per_tok=8, moe_intermediate_size=2560,
            shared_expert_intermediate_size=20480, max_window_layers=28)
SIZES = {"a2.7b": ("Qwen1.5-MoE-A2.7B", A27B), "57b-a14b": ("Qwen2-57B-A14B", A14B)}
PUBLISHED_DECODE_B1 = 37.0          # the reference's only Qwen2-MoE number: "~37 tok/s", batch 1, FP16, RTX A6000


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            j = json.load(f)
        return {"hbm_gbs": j["hbm_gbs"], "bf16_tflops": j["bf16_tflops"],
                "bf16_tflops_sustained": j.get("bf16_tflops_sustained", j["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, device=0):
        self.device = device
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = sorted(float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit())
        mx = [float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[3 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


def weight_bytes_decode(cfg, layers, distinct_experts_per_layer, item=2):
    """Bytes of weights one decode step reads: every matrix it uses once."""
    H, d = cfg["hidden_size"], cfg["hidden_size"] // cfg["num_attention_heads"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    mI, sI, E, V = cfg["moe_intermediate_size"], cfg["shared_expert_intermediate_size"], cfg["num_experts"], cfg["vocab_size"]
    attn = (nh + 2 * nkv) * d * H + (nh + 2 * nkv) * d + nh * d * H
    norms = 2 * H
    router = (E + 1) * H
    shared = 3 * sI * H
    per_expert = 3 * mI * H
    total = 0
    for n_exp in distinct_experts_per_layer:
        total += attn + norms + router + shared + n_exp * per_expert
    total += H + V * H            # final norm, output head (the embedding rows read are negligible)
    return total * item


def prefill_flops(cfg, layers, T):
    """Multiply-add flops (2 per MAC) of one whole prompt of T tokens, logits at the last row."""
    H, d = cfg["hidden_size"], cfg["hidden_size"] // cfg["num_attention_heads"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    mI, sI, E, K, V = (cfg["moe_intermediate_size"], cfg["shared_expert_intermediate_size"], cfg["num_experts"],
                       cfg["num_experts_per_tok"], cfg["vocab_size"])
    per_tok = 2 * ((nh + 2 * nkv) * d * H + nh * d * H + (E + 1) * H + 3 * sI * H + K * 3 * mI * H)
    attn = 2 * 2 * nh * d * (T * (T + 1) // 2)           # QK^T and PV over the causal half
    return layers * (per_tok * T + attn) + 2 * V * H


def run_timeline(args):
    """``--timeline``: the kernels of one step as they run inside the engine (CUPTI through torch.profiler:
    real overlap between streams, CUDA-graph replays for decode), aggregated by kernel and, for one layer,
    in time order.  Prints text, not the JSON line; nothing here is a benchmark value."""
    import collections
    import torch
    from torch.profiler import ProfilerActivity, profile
    from mini_infer_b200.engine.defaults import DEFAULT_PAGE_SIZE
    from mini_infer_b200.engine.loading import random_model
    from mini_infer_b200.engine.step import ModelRunner, StepEntry

    model_name, named = SIZES[args.sizes]
    cfg = dict(named)
    cfg["num_hidden_layers"] = args.layers if args.layers > 0 else 4
    model, rt = random_model(cfg, seed=args.seed, dtype="bfloat16", device="cuda:0")
    page, B, T = DEFAULT_PAGE_SIZE, args.batch, args.prompt_len
    decode = args.only != "prefill"
    runner = ModelRunner(model, rt, page_size=page, num_pages=(B if decode else 2) * (T // page + 8),
                         max_requests=max(B, 2), max_tokens_per_step=max(T, B), max_context=args.context,
                         cuda_graphs=not args.eager)
    g = torch.Generator().manual_seed(args.seed)

    def prompt():
        return torch.randint(0, cfg["vocab_size"], (T,), generator=g).tolist()

    if decode:
        for b in range(B):
            runner.add_request(b)
            runner.step([StepEntry(b, prompt(), [])])
        state = {"toks": [1] * B}

        def step():
            res = runner.step([StepEntry(b, [state["toks"][b]], [0]) for b in range(B)])
            state["toks"] = res.logits.argmax(-1).tolist()
        first_kernel, layer_mark = "embed_gather", ("qkv_skinny", "qkv_post")
    else:
        count = {"n": 0}

        def step():
            count["n"] += 1
            runner.add_request(("p", count["n"]))
            runner.step([StepEntry(("p", count["n"]), prompt(), [T - 1])])
            runner.release(("p", count["n"]))
        first_kernel, layer_mark = "embed_gather", ("qkv_post", "qkv_skinny")
    for _ in range(4):
        step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(2):
            step()
        torch.cuda.synchronize()
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and e.name
           and "Memcpy" not in e.name and "Memset" not in e.name]
    evs.sort(key=lambda e: e.time_range.start)
    starts = [i for i, e in enumerate(evs) if first_kernel in e.name]
    sel = evs[starts[-1]:]
    t0, last_end, idle = sel[0].time_range.start, sel[0].time_range.start, 0.0
    agg = collections.OrderedDict()
    for e in sel:
        s_, e_ = e.time_range.start, e.time_range.end
        idle += max(0.0, s_ - last_end)
        last_end = max(last_end, e_)
        a = agg.setdefault(e.name[:90], [0, 0.0])
        a[0] += 1
        a[1] += e_ - s_
    what = f"decode step, batch {B}, context {T}" if decode else f"prefill of {T} tokens"
    print(f"{what}, {cfg['num_hidden_layers']} layers of {model_name} size: {last_end - t0:.1f} us from the first "
          f"kernel's start to the last one's end, {idle:.1f} us with no kernel running, {len(sel)} kernels")
    for n, (c, d) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
        print(f"{d:9.1f} us x{c:<4} {n}")
    marks = [i for i, e in enumerate(sel) if any(m in e.name for m in layer_mark)]
    if len(marks) >= 3:
        a, b = marks[1] - 1, marks[2] - 1
        base = sel[a].time_range.start
        print("one layer in time order (start, duration):")
        for e in sel[a:b]:
            print(f"  +{e.time_range.start - base:7.1f}  {e.time_range.end - e.time_range.start:6.1f} us  {e.name[:80]}")
    return 0


def run_serving(args):
    """A continuous-batching workload through ``LLM.generate``, in the manner of the reference's
    ``benchmarks/bench_continuous.cpp`` (requests of mixed prompt lengths submitted at once, a fixed number of
    new tokens each) with seeded synthetic token ids: throughput and time to first token, cold (the first
    call captures its CUDA graphs) and warm."""
    import torch
    from mini_infer_b200.engine.defaults import DEFAULT_PAGE_SIZE
    from mini_infer_b200.engine.llm import LLM
    from mini_infer_b200.engine.loading import random_model
    from mini_infer_b200.sampling import SamplingParams
    model_name, named = SIZES[args.sizes]
    cfg = dict(named)
    full_layers = named["num_hidden_layers"]
    cfg["num_hidden_layers"] = args.layers if args.layers > 0 else full_layers
    model, rt = random_model(cfg, seed=args.seed, dtype="bfloat16", device="cuda:0")
    g = torch.Generator().manual_seed(args.seed + 3)
    n, new = args.serving, args.serving_new_tokens
    lo, hi = args.serving_prompt_min, args.serving_prompt_max
    lens = torch.randint(lo, hi + 1, (n,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (k,), generator=g).tolist() for k in lens]
    ctx = hi + new + 16
    llm = LLM(model, runtime=rt, max_seq_len=ctx, max_running=args.serving_max_running, max_tokens_per_step=2048,
              prefill_chunk=2048, num_pages=args.serving_max_running * (ctx // DEFAULT_PAGE_SIZE + 1))
    sp = SamplingParams(greedy=True, max_new_tokens=new)
    llm.generate(prompts[:2], SamplingParams(greedy=True, max_new_tokens=4))       # library warm-up only
    runs = []
    for _ in range(3):
        torch.cuda.synchronize()
        t0 = time.time()
        outs = llm.generate(prompts, sp)
        torch.cuda.synchronize()
        dt = time.time() - t0
        ttft = sorted(o.ttft for o in outs if o.ttft is not None)
        h = llm.last_history
        runs.append({"seconds": round(dt, 3), "out_tok_s": round(n * new / dt, 1),
                     "total_tok_s": round((sum(lens) + n * new) / dt, 1),
                     "ttft_ms_p50": round(1e3 * ttft[len(ttft) // 2], 1), "ttft_ms_max": round(1e3 * ttft[-1], 1),
                     "steps": len(h), "steps_with_prompt_and_decode": sum(1 for s in h if s.prefill_tokens and s.decode_tokens),
                     "graphs": len(llm.runner._graphs)})
    print(json.dumps({"impl": "ours", "workload": "continuous batching, all requests submitted at once",
                      "model": f"{model_name} layer sizes", "layers": cfg["num_hidden_layers"], "requests": n,
                      "prompt_tokens": sum(lens), "prompt_len_range": [lo, hi], "new_tokens_each": new,
                      "max_running": args.serving_max_running, "cold": runs[0], "warm": runs[-1],
                      "data": "synthetic: random-init weights, seeded uniform-random token ids"}))
    return 0


def run_ours(args):
    import torch
    from mini_infer_b200.engine.llm import LLM, GPUExecutor
    from mini_infer_b200.engine.loading import random_model
    from mini_infer_b200.engine.request import Request
    from mini_infer_b200.engine.scheduler import Scheduler, SchedulerConfig
    from mini_infer_b200.engine.step import ModelRunner, StepEntry
    from mini_infer_b200.engine.defaults import DEFAULT_PAGE_SIZE
    from mini_infer_b200.ops.library import launch_count
    from mini_infer_b200.sampling import SamplingParams
    from mini_infer_b200.sampling.sampler import Sampler

    pk = peaks()
    model_name, named = SIZES[args.sizes]
    cfg = dict(named)
    full_layers = named["num_hidden_layers"]
    if args.layers <= 0:
        args.layers = full_layers
    cfg["num_hidden_layers"] = args.layers
    dev = "cuda:0"
    t0 = time.time()
    model, rt = random_model(cfg, seed=args.seed, dtype="bfloat16", device=dev)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    page = DEFAULT_PAGE_SIZE
    prompt_len, ctx_len = args.prompt_len, args.context
    if args.only != "all":
        args.points = False
    point_max = max([int(x) for x in args.point_batches.split(",") if x] or [1])
    max_b = max(args.batch, point_max if args.points else args.batch, 1)
    per_req_tokens = prompt_len + args.steps + args.warmup + 2 * max_b + 16
    num_pages = max_b * (-(-per_req_tokens // page)) + 8
    llm = LLM(model, runtime=rt, max_seq_len=ctx_len, page_size=page, num_pages=num_pages, max_running=max_b,
              max_tokens_per_step=max(2048, max_b, prompt_len), prefill_chunk=max(2048, prompt_len),
              cuda_graphs=not args.eager)
    runner, sampler = llm.runner, llm.sampler
    g = torch.Generator().manual_seed(args.seed)

    def random_prompt(n):
        return torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()

    def time_events(fn):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    # ---- prefill: one request of prompt_len tokens, logits at the last row ------------------- #
    def prefill_once():
        runner.add_request("pf")
        toks = random_prompt(prompt_len)
        ms = time_events(lambda: runner.step([StepEntry("pf", toks, [prompt_len - 1])]))
        runner.release("pf")
        return ms
    prefill = None
    if args.only in ("all", "prefill"):
        for _ in range(2):
            prefill_once()
        if args.profiler_range:
            torch.cuda.profiler.start()
        pf_ms = min(prefill_once() for _ in range(1 if args.profiler_range else 3))
        if args.profiler_range:
            torch.cuda.profiler.stop()
        pf_flops = prefill_flops(cfg, args.layers, prompt_len)
        prefill = {"value": round(prompt_len / (pf_ms / 1e3), 1), "tokens": prompt_len, "ms": round(pf_ms, 3),
                   "frac": round(pf_flops / (pf_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                   "tflops": round(pf_flops / (pf_ms / 1e3) / 1e12, 2), "of": pk["source"]}
    if args.only == "prefill":
        print(json.dumps({"impl": "ours", "only": "prefill", "layers": args.layers, "prefill": prefill}))
        return 0

    # ---- decode through the scheduler (what the Python entry point drives) -------------------- #
    def decode_run(batch, steps, warmup, clocks=False):
        ex = GPUExecutor(runner, sampler)
        sched = Scheduler(ex, SchedulerConfig(max_tokens_per_step=max(2048, batch, prompt_len), max_running=batch,
                                              prefill_chunk=2048, max_context=ctx_len))
        sp = SamplingParams(greedy=True, max_new_tokens=steps + warmup + 2 * batch + 8)   # early requests decode
        # while later prompts are still being prefilled
        for i in range(batch):
            sched.submit(Request(("bench", batch, i), random_prompt(prompt_len), sp, stream=i))
        while any(r.remaining > 1 for r in sched.running) or sched.waiting:     # untimed prefill
            sched.step()
        for _ in range(warmup):
            sched.step()
        sampler_clock = ClockSampler() if clocks else None
        if sampler_clock:
            sampler_clock.start()
        torch.cuda.synchronize()
        if clocks and args.profiler_range:
            torch.cuda.profiler.start()
        launches0 = launch_count() + runner.graph_kernel_launches
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.perf_counter()
        a.record()
        for _ in range(steps):
            st = sched.step()
            assert st.decode_tokens == batch and st.prefill_tokens == 0
        b.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - w0
        dev_ms = a.elapsed_time(b)
        if clocks and args.profiler_range:
            torch.cuda.profiler.stop()
        launches = launch_count() + runner.graph_kernel_launches - launches0   # eager + replayed in graphs
        clock = sampler_clock.stop() if sampler_clock else None
        kv_tokens = sum(r.num_computed for r in sched.running)
        for r in list(sched.running):
            sched._finish(r, "length")
        return {"dev_ms": dev_ms, "wall_s": wall, "launches": launches, "clock": clock, "kv_tokens": kv_tokens}

    main = decode_run(args.batch, args.steps, args.warmup, clocks=True)
    ms_per_step = main["dev_ms"] / args.steps
    value = args.batch * args.steps / (main["dev_ms"] / 1e3)
    if args.only == "decode":
        print(json.dumps({"impl": "ours", "only": "decode", "layers": args.layers, "batch": args.batch,
                          "ms_per_step": round(ms_per_step, 4), "value": round(value, 1)}))
        return 0

    # ---- the same through the Python entry point: host token ids in, host token ids out ------- #
    prompts = [random_prompt(prompt_len) for _ in range(args.batch)]

    def generate_seconds(new_tokens):
        torch.cuda.synchronize()
        t = time.perf_counter()
        outs = llm.generate(prompts, SamplingParams(greedy=True, max_new_tokens=new_tokens))
        dt = time.perf_counter() - t
        assert all(len(o.token_ids) == new_tokens for o in outs)
        return dt
    # Two calls that differ by `steps` new tokens per request; both hold the same prefill, the same
    # staggered start (a prompt per step) and the same tail in which the first requests have ended, so
    # their difference is `steps` decode steps of the full batch.
    head = 2 * args.batch
    generate_seconds(2)                                            # warm-up of this path
    t_short = min(generate_seconds(head) for _ in range(3))
    t_long = min(generate_seconds(args.steps + head) for _ in range(3))
    e2e_value = args.batch * args.steps / max(t_long - t_short, 1e-9)

    # ---- roofline of the decode step ----------------------------------------------------------- #
    E, K = cfg["num_experts"], cfg["num_experts_per_tok"]
    expected_distinct = E * (1.0 - (1.0 - K / E) ** args.batch)
    wbytes = weight_bytes_decode(cfg, args.layers, [expected_distinct] * args.layers)
    d = cfg["hidden_size"] // cfg["num_attention_heads"]
    kv_bytes = main["kv_tokens"] * args.layers * 2 * cfg["num_key_value_heads"] * d * 2
    achieved = (wbytes + kv_bytes) / (ms_per_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(wbytes + kv_bytes),
                "of": pk["source"]}

    points = {}
    if args.points:
        for b, key in ((int(x), f"decode_b{int(x)}") for x in args.point_batches.split(",") if x):
            r = decode_run(b, max(4, args.steps // 2), 3)
            points[key] = round(b * max(4, args.steps // 2) / (r["dev_ms"] / 1e3), 1)

    staging_bytes = runner._host.numel() * 4
    out = {
        "metric": f"decode tok/s at batch {args.batch} ({model_name} sizes, {prompt_len}-token prompts)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(points.get("decode_b1", 0.0) / PUBLISHED_DECODE_B1, 2)
        if points and args.sizes == "a2.7b" else None,
        "dtype": "bf16", "data": "synthetic: random-init weights, seeded uniform-random token ids",
        "impl": "ours",
        "config": {"model": f"{model_name} layer sizes (Qwen2MoeForCausalLM)", "global_batch": args.batch,
                   "seq_len": prompt_len, "context": ctx_len, "parallelism": "single GPU",
                   "layers": args.layers, "layers_of_named_config": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"], "experts": cfg["num_experts"],
                   "top_k": cfg["num_experts_per_tok"], "moe_intermediate": cfg["moe_intermediate_size"],
                   "shared_intermediate": cfg["shared_expert_intermediate_size"], "vocab": cfg["vocab_size"],
                   "page_size": page,
                   "l2": "every step reads GBs of weights (inputs larger than L2)",
                   "vs_baseline_note": "decode_b1 / the reference's ~37 tok/s (batch 1, FP16, RTX A6000)"},
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": staging_bytes,
                "d2h_bytes_per_step": args.batch * 4},
        "gpu_launches": main["launches"],
        "clocks": main["clock"],
        "prefill": prefill, "roofline": roofline, "points": points,
        "load_seconds": round(load_s, 1),
    }
    print(json.dumps(out))
    return 0


# --------------------------------------------------------------------------- #
# --vizalix: the Vizalix design beside the closest built-in model at equal sizes
# --------------------------------------------------------------------------- #
VIZALIX_SIZES = {          # width, heads, key/value heads, head size, feed-forward width
    "0.3b": (1024, 8, 4, 128, 2816),
    "1b": (2048, 16, 4, 128, 5632),
    "3b": (3072, 24, 8, 128, 8192),
}


def vizalix_config(size, window, vocab):
    W, H, G, d, ff = VIZALIX_SIZES[size]
    mlp = {"kind": "dense", "ff": ff}
    delta = {"type": "channel_delta", "mlp": mlp,
             "mixer": {"heads": H, "kv_heads": H, "dim": d, "vdim": d, "conv": 4, "decay_rank": 64, "gate_rank": 64}}
    attn = {"type": "attention", "mlp": mlp,
            "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "mask": {"size": window}, "scale": d ** -0.5,
                      "softcap": 50.0, "rot": {"base": 500000.0, "dims": d // 2,
                                               "scaling": {"factor": 4.0, "low": 1.0, "high": 8.0, "original": 8192}}}}
    mamba = {"type": "mamba2", "mlp": mlp,
             "mixer": {"heads": 2 * H, "vdim": d // 2, "state": 128, "groups": 1, "norm_groups": 1, "conv": 4}}
    return {"architecture": "Vizalix", "vocab": vocab, "width": W, "norm": {"eps": 1e-6},
            "layers": [delta, attn, mamba, delta, attn, mamba], "loop": {"start": 1, "stop": 5, "times": 2}}


def dense_twin_config(size, window, vocab, layer_runs):
    """The closest built-in model: Qwen2-MoE with every layer dense (grouped-query attention behind the same
    window, SwiGLU feed-forward), as many layers as the Vizalix model has layer runs, the same widths."""
    W, H, G, d, ff = VIZALIX_SIZES[size]
    return dict(A27B, vocab_size=vocab, hidden_size=W, intermediate_size=ff, num_hidden_layers=layer_runs,
                num_attention_heads=H, num_key_value_heads=G, head_dim=d, num_experts=4, num_experts_per_tok=2,
                moe_intermediate_size=64, shared_expert_intermediate_size=0, mlp_only_layers=list(range(layer_runs)),
                use_sliding_window=True, sliding_window=window, max_window_layers=0, max_position_embeddings=1 << 20)


def _kernel_table(step, steps=2):
    """Device time per kernel of ``steps`` calls of ``step`` (CUPTI through torch.profiler), per call."""
    import collections
    import torch
    from torch.profiler import ProfilerActivity, profile
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            step()
        torch.cuda.synchronize()
    agg = collections.OrderedDict()
    for e in prof.events():
        if e.device_type != torch.autograd.DeviceType.CUDA or not e.name or "Memcpy" in e.name or "Memset" in e.name:
            continue
        name = e.name.split("<")[0].split("(")[0].replace("void ", "").replace("mi::", "")[:60]
        a = agg.setdefault(name, [0, 0.0])
        a[0] += 1
        a[1] += e.time_range.end - e.time_range.start
    return {n: {"launches": c // steps, "us": round(d / steps, 1)} for n, (c, d) in
            sorted(agg.items(), key=lambda kv: -kv[1][1])}


def _vizalix_kernel_work(cfg, T, B, ctx, decode):
    """Algorithmic bytes and floating-point operations of the design's own kernels for one step over all
    layer runs (prefill of T tokens of one request, or a decode step of B requests at context ctx)."""
    runs = {0: 1, 1: 2, 2: 2, 3: 2, 4: 2, 5: 1}
    rows = B if decode else T
    W = cfg["width"]
    out = {}

    def add(name, by, fl):
        a = out.setdefault(name, [0.0, 0.0])
        a[0] += by
        a[1] += fl
    for i, L in enumerate(cfg["layers"]):
        n, m = runs[i], L["mixer"]
        if L["type"] == "channel_delta":
            H, d, e = m["heads"], m["dim"], m["vdim"]
            ch = 2 * m["kv_heads"] * d + H * e
            state = (B if decode else 1) * H * d * e * 4 * 2
            add("delta_scan_kernel", n * (rows * (ch + H * d + H + H * e) * 4 + state), n * rows * H * d * e * 6.0)
            for name in ("causal_conv_silu_kernel", "causal_conv_silu_vec4_kernel"):
                add(name, n * rows * ch * 8, n * rows * ch * 8.0)
            add("gated_group_rmsnorm_kernel", n * rows * H * e * (4 + 4 + 2), 0)
        elif L["type"] == "mamba2":
            H, P, N = m["heads"], m["vdim"], m["state"]
            ch = H * P + 2 * N
            state = (B if decode else 1) * H * N * P * 4 * 2
            add("ssd_scan_kernel", n * (rows * (ch + H + H * P) * 4 + state), n * rows * H * N * P * 4.0)
            for name in ("causal_conv_silu_kernel", "causal_conv_silu_vec4_kernel"):
                add(name, n * rows * ch * 8, n * rows * ch * 8.0)
            add("gated_group_rmsnorm_kernel", n * rows * H * P * (4 + 4 + 2), 0)
        else:
            H, G, d, e, win = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["mask"]["size"]
            if decode:
                keys = min(ctx, win)
                pairs = B * keys
                by = B * keys * G * (d + e) * 2 + B * H * (d + e) * 2
            else:
                pairs = sum(min(t + 1, win) for t in range(T))
                by = T * (H * (d + e) + G * (d + e)) * 2
            for name in ("attn_mix_kernel", "attn_mix_tc_kernel"):       # whichever form the sizes take
                add(name, n * by, n * pairs * H * (2.0 * d + 2.0 * e + 2.0 * H))
            add("rope_store_kernel", n * rows * (H * d + G * (d + e)) * 6, 0)
        add("add2_rmsnorm_scalar_kernel", n * rows * W * (4 * 4 + 2 * 2), 0)
        for name in ("geglu_tanh_kernel", "geglu_tanh_bf16x8_kernel"):
            add(name, n * rows * L["mlp"]["ff"] * 6, 0)
    return out


def _twin_kernel_work(size, window, T, B, ctx, decode, layers):
    """The same for the like kernels of the dense twin: attention, the two norms, the gated activation."""
    W, H, G, d, ff = VIZALIX_SIZES[size]
    rows = B if decode else T
    if decode:
        keys = min(ctx, window)
        pairs, by = B * keys, B * keys * G * 2 * d * 2 + B * H * 2 * d * 2
        attn = "attn_decode_split_kernel"
    else:
        pairs = sum(min(t + 1, window) for t in range(T))
        by, attn = T * (H + G) * 2 * d * 2, "pt::attn_prefill_tc_kernel"
    return {attn: [layers * by, layers * pairs * H * 4.0 * d],
            "add_rmsnorm_vec_kernel": [(2 * layers + 1) * rows * W * (3 * 4 + 2), 0.0],
            "swiglu_bf16x8_kernel": [layers * rows * ff * 6, 0.0],
            "qkv_post_rows_kernel": [layers * rows * (H + 2 * G) * d * 6, 0.0]}


def run_vizalix(args):
    return _run_design(args, "vizalix", args.vizalix, args.vizalix_window,
                       lambda size, window, vocab: vizalix_config(size, window, vocab),
                       lambda size, window, vocab: dense_twin_config(size, window, vocab, 10),
                       _vizalix_kernel_work,
                       lambda cfg, size, window, T, B, ctx, dec: _twin_kernel_work(size, window, T, B, ctx, dec, 10),
                       "dense_twin")


def _run_design(args, design, sizes, window, make_config, make_twin, design_work, twin_work, twin_name,
                graph_prompts=False):
    """A design beside the closest built-in model: prefill and decode throughput at sizes that resemble a real
    model's layers (random weights), with the device time of every kernel of one step of each and, for the
    kernels that the work functions name, the share of the roofline (the slower of algorithmic bytes over the
    measured copy bandwidth and operations over the measured bf16 product rate).  Prints one JSON line; the
    default workload of this file is not touched.  ``graph_prompts``: the prompt's step is replayed from a
    captured pass, as the engine does for the full portions of a long prompt (a step of a small model is
    otherwise bound by the host's launches, not by the device)."""
    import torch
    from mini_infer_b200.engine.defaults import DEFAULT_PAGE_SIZE
    from mini_infer_b200.engine.loading import random_model
    from mini_infer_b200.engine.step import ModelRunner, StepEntry

    pk = peaks()
    T, B, ctx, page = args.prompt_len, args.batch, args.prompt_len, DEFAULT_PAGE_SIZE
    vocab = 32000
    result = {"metric": f"{design}_vs_{twin_name}", "prompt_len": T, "decode_batch": B, "decode_context": ctx,
              "window": window, "dtype": "bf16", "data": "synthetic", "peaks": pk, "sizes": {}}
    sampler = ClockSampler()
    sampler.start()
    for size in [x for x in sizes.split(",") if x]:
        entry = {}
        for which, cfg in ((design, make_config(size, window, vocab)), (twin_name, make_twin(size, window, vocab))):
            model, rt = random_model(cfg, seed=args.seed, dtype="bfloat16", device="cuda:0")
            runner = ModelRunner(model, rt, page_size=page, num_pages=(B + 1) * (-(-(ctx + 512) // page)) + 8,
                                 max_requests=max(B, 2), max_tokens_per_step=max(T, B), max_context=ctx + 512,
                                 cuda_graphs=not args.eager, graph_chunk_tokens=T if graph_prompts and not args.eager else 0)
            g = torch.Generator().manual_seed(args.seed)
            V = cfg.get("vocab", cfg.get("vocab_size"))

            def prompt():
                return torch.randint(0, V, (T,), generator=g).tolist()

            def timed(fn, reps):
                best = 1e30
                for _ in range(reps):
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize()
                    a.record()
                    fn()
                    b.record()
                    torch.cuda.synchronize()
                    best = min(best, a.elapsed_time(b))
                return best

            count = {"n": 0}

            def prefill():
                count["n"] += 1
                rid = ("p", count["n"])
                runner.add_request(rid)
                runner.step([StepEntry(rid, toks, [T - 1])])
                runner.release(rid)
            toks = prompt()
            for _ in range(max(3, args.warmup)):
                prefill()
            pf_ms = timed(prefill, 5)
            pf_kernels = _kernel_table(prefill)
            for b in range(B):
                runner.add_request(b)
                runner.step([StepEntry(b, prompt(), [])])
            # a token of its own for every request: rows that are all alike would all pick the same experts
            state = {"toks": torch.randint(0, V, (B,), generator=g).tolist()}

            def decode():
                res = runner.step([StepEntry(b, [state["toks"][b]], [0]) for b in range(B)])
                state["last"] = res.logits
            for _ in range(max(3, args.warmup)):
                decode()

            def decode_many():
                for _ in range(args.steps):
                    decode()
            dc_ms = timed(decode_many, 2) / args.steps
            dc_kernels = _kernel_table(decode, 4)
            entry[which] = {"prefill_tok_s": round(T / (pf_ms / 1e3), 1), "prefill_ms": round(pf_ms, 3),
                            "decode_tok_s": round(B / (dc_ms / 1e3), 1), "decode_ms_per_step": round(dc_ms, 4),
                            "params_millions": round(sum(p.numel() for part in model.all_parts() for p in
                                                         vars(part).values() if isinstance(p, torch.Tensor)
                                                         and p.dtype == torch.bfloat16) / 1e6, 1),
                            "prefill_kernels": pf_kernels, "decode_kernels": dc_kernels}
            if True:
                for phase, table, dec in (("prefill", pf_kernels, False), ("decode", dc_kernels, True)):
                    work = (design_work(cfg, T, B, ctx, dec) if which == design
                            else twin_work(cfg, size, window, T, B, ctx, dec))
                    for name, (by, fl) in work.items():
                        if name in table:
                            floor_us = max(by / (pk["hbm_gbs"] * 1e9), fl / (pk["bf16_tflops"] * 1e12)) * 1e6
                            table[name]["roofline_us"] = round(floor_us, 2)
                            table[name]["frac"] = round(floor_us / max(table[name]["us"], 1e-9), 4)
            del runner, model
            torch.cuda.empty_cache()
        result["sizes"][size] = entry
    result["clocks"] = sampler.stop()
    print(json.dumps(result))
    return 0



# --------------------------------------------------------------------------- #
# --nipapel: the Nipapel design beside the closest built-in model (Qwen2-MoE) at equal sizes
# --------------------------------------------------------------------------- #
NIPAPEL_SIZES = {   # width, heads, key/value heads, head size, latent size, rotated size, query latent, latent heads'
                    # unrotated size and value size, dense feed-forward, experts, experts per token, expert width
    "0.5b": (1024, 8, 2, 128, 128, 32, 384, 64, 64, 2816, 16, 2, 1024),
    "a2.7b": (2048, 16, 4, 128, 128, 64, 768, 64, 64, 5632, 60, 4, 1408),
}
NIPAPEL_LAYERS = 6


def nipapel_config(size, window, vocab):
    W, H, G, d, c, r, qr, dl, el, ff, E, K, eff = NIPAPEL_SIZES[size]
    dense = {"kind": "dense", "ff": ff, "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": eff, "limit": 7.0}, "router": {"experts": E, "top": K}}
    attn = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "mask": {"size": window, "keep_first": 4},
            "rot": {"base": 500000.0, "dims": d // 2}, "scale": d ** -0.5}

    def latent(kv_from=None):
        m = {"heads": H, "dim": dl, "rot_dim": r, "vdim": el, "kv_rank": c, "q_rank": qr, "mask": {"size": window},
             "rot": {"base": 10000.0, "dims": r}, "scale": (dl + r) ** -0.5}
        if kv_from is not None:
            m["kv_from"] = kv_from
        return m
    layers = [{"type": "attention", "mixer": attn, "mlp": dense},
              {"type": "latent_attention", "mixer": latent(), "mlp": moe},
              {"type": "latent_attention", "mixer": latent(1), "mlp": moe},
              {"type": "attention", "mixer": attn, "mlp": moe},
              {"type": "latent_attention", "mixer": latent(), "mlp": moe},
              {"type": "latent_attention", "mixer": latent(4), "mlp": moe}]
    return {"architecture": "Nipapel", "vocab": vocab, "width": W, "norm": {"eps": 1e-6}, "layers": layers}


def moe_twin_config(size, window, vocab):
    """The closest built-in model: Qwen2-MoE with the same width, heads, window, experts and expert width, a
    dense first layer of the same feed-forward width, no shared expert, as many layers."""
    W, H, G, d, c, r, qr, dl, el, ff, E, K, eff = NIPAPEL_SIZES[size]
    return dict(A27B, vocab_size=vocab, hidden_size=W, intermediate_size=ff, num_hidden_layers=NIPAPEL_LAYERS,
                num_attention_heads=H, num_key_value_heads=G, head_dim=d, num_experts=E, num_experts_per_tok=K,
                moe_intermediate_size=eff, shared_expert_intermediate_size=0, mlp_only_layers=[0],
                norm_topk_prob=True, use_sliding_window=True, sliding_window=window, max_window_layers=0,
                max_position_embeddings=1 << 20)


def _nipapel_kernel_work(cfg, T, B, ctx, decode):
    """Algorithmic bytes and floating-point operations of the design's own kernels for one step over all layers
    (prefill of T tokens of one request, or a decode step of B requests at context ctx)."""
    rows = B if decode else T
    out = {}
    # decode steps take the split kernel; prompt portions the tensor-memory attention where the sizes allow
    attention_kernels = ("attn_mix_tc_kernel",) if decode else ("attn_mix_tc_kernel", "pt::attn_prefill_tc_kernel")

    def add(name, by, fl):
        a = out.setdefault(name, [0.0, 0.0])
        a[0] += by
        a[1] += fl
    for L in cfg["layers"]:
        m = L["mixer"]
        win = m["mask"]["size"]
        keys = min(ctx, win) + m["mask"].get("keep_first", 0)
        pairs = B * keys if decode else sum(min(t + 1, win) for t in range(T))
        if L["type"] == "attention":
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            by = (B * keys * G * (d + e) * 2 + B * H * (d + e) * 2) if decode else T * (H + G) * (d + e) * 2
            for name in attention_kernels:
                add(name, by, pairs * H * (2.0 * d + 2.0 * e))
            add("rope_store_kernel", rows * (H * d + G * (d + e)) * 6, 0)
        else:
            H, d, r, e, c = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            by = (B * keys * (c + r) * 2 + B * H * (2 * c + r) * 2) if decode else T * (H * (2 * c + r) + c + r) * 2
            for name in attention_kernels:
                add(name, by, pairs * H * (2.0 * (c + r) + 2.0 * c))
            if m.get("kv_from") is None:
                add("latent_store_kernel", rows * (c + r) * 6, 0)
            add("latent_query_kernel", rows * H * ((d + r) * 4 + (d + r) * 2), 0)
            add("sigmoid_gate_kernel", rows * H * e * (2 + 4 + 2), 0)
        if L["mlp"]["kind"] == "dense":
            add("clamped_glu_kernel", rows * L["mlp"]["ff"] * (8 + 2), 0)
    return out


def _moe_twin_kernel_work(cfg, size, window, T, B, ctx, decode):
    W, H, G, d = NIPAPEL_SIZES[size][:4]
    ff = NIPAPEL_SIZES[size][9]
    rows, layers = (B if decode else T), NIPAPEL_LAYERS
    if decode:
        keys = min(ctx, window)
        pairs, by = B * keys, B * keys * G * 2 * d * 2 + B * H * 2 * d * 2
        attn = "attn_decode_split_kernel"
    else:
        pairs = sum(min(t + 1, window) for t in range(T))
        by, attn = T * (H + G) * 2 * d * 2, "pt::attn_prefill_tc_kernel"
    return {attn: [layers * by, layers * pairs * H * 4.0 * d],
            "swiglu_bf16x8_kernel": [rows * ff * 6, 0.0],
            "qkv_post_rows_kernel": [layers * rows * (H + 2 * G) * d * 6, 0.0]}


def run_nipapel(args):
    return _run_design(args, "nipapel", args.nipapel, args.nipapel_window, nipapel_config, moe_twin_config,
                       _nipapel_kernel_work, _moe_twin_kernel_work, "moe_twin", graph_prompts=True)


# --------------------------------------------------------------------------- #
# --tofinex: the Tofinex design beside the closest built-in model (Qwen2-MoE) at equal sizes
# --------------------------------------------------------------------------- #
TOFINEX_SIZES = {   # width, heads, key/value heads, head size, dense feed-forward, experts, experts per token, expert
                    # width, shared expert width
    "0.5b": (1024, 8, 2, 128, 2816, 16, 2, 1024, 2816),
    "a2.7b": (2048, 16, 4, 128, 5632, 60, 4, 1408, 5632),      # the layer sizes of Qwen1.5-MoE-A2.7B
}
TOFINEX_LAYERS = 6


def tofinex_config(size, window, vocab):
    W, H, G, d, ff, E, K, eff, sff = TOFINEX_SIZES[size]
    attn = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "rot": {"base": 500000.0, "dims": d}, "scale": d ** -0.5,
            "softcap": 30.0, "v_mix": True}
    moe = {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": E, "top": K}, "shared": {"ff": sff}}
    layers = [{"type": "attention", "mixer": attn, "mlp": {"kind": "dense", "ff": ff} if i == 0 else moe}
              for i in range(TOFINEX_LAYERS)]
    return {"architecture": "Tofinex", "vocab": vocab, "width": W, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "logit_softcap": 30.0, "layers": layers}


def tofinex_twin_config(size, window, vocab):
    """The closest built-in model: Qwen2-MoE with the same width, heads, experts, expert and shared expert
    widths, a dense first layer of the same feed-forward width, attention over all earlier tokens, as many
    layers."""
    W, H, G, d, ff, E, K, eff, sff = TOFINEX_SIZES[size]
    return dict(A27B, vocab_size=vocab, hidden_size=W, intermediate_size=ff, num_hidden_layers=TOFINEX_LAYERS,
                num_attention_heads=H, num_key_value_heads=G, head_dim=d, num_experts=E, num_experts_per_tok=K,
                moe_intermediate_size=eff, shared_expert_intermediate_size=sff, mlp_only_layers=[0],
                norm_topk_prob=False, use_sliding_window=False, max_position_embeddings=1 << 20)


def _tofinex_kernel_work(cfg, T, B, ctx, decode):
    """Algorithmic bytes and floating-point operations of the design's own kernels for one step over all layers
    (prefill of T tokens of one request, or a decode step of B requests at context ctx)."""
    rows, W = (B if decode else T), cfg["width"]
    out = {}

    def add(name, by, fl):
        a = out.setdefault(name, [0.0, 0.0])
        a[0] += by
        a[1] += fl
    for L in cfg["layers"]:
        m = L["mixer"]
        H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        pairs = B * ctx if decode else T * (T + 1) // 2
        by = (B * ctx * G * (d + e) * 2 + B * H * (d + e) * 2) if decode else T * (H + G) * (d + e) * 2
        for name in (("attn_mix_tc_kernel", "attn_decode_split_kernel") if decode
                     else ("attn_mix_tc_kernel", "pt::attn_prefill_tc_kernel")):
            add(name, by, pairs * H * (2.0 * d + 2.0 * e))
        # float32 rows in (and the first layer's values once more), queries out, keys and values into the cache
        for name in ("rope_store_kernel", "rope_store_vec_kernel"):
            add(name, rows * ((H * d + G * (d + e)) * 6 + G * e * 4), 0)
        # a part's float32 output in, the residual read and written, its rounded copy written
        parts = 1 if L["mlp"] is None else 2
        for name in ("out_norm_add_kernel", "out_norm_add_vec_kernel"):
            add(name, parts * rows * W * (4 + 8 + 2), 0)
            if L["mlp"] is not None and L["mlp"]["kind"] == "moe":
                K = L["mlp"]["router"]["top"]
                # the experts' rows and the shared expert's row (float32) join the out_norm_add above
                add(name, rows * W * 4 * K, 0)
        if L["mlp"] is not None and L["mlp"]["kind"] == "moe":
            K = L["mlp"]["router"]["top"]
            add("tc::gather_rows_kernel", rows * W * 2 * (1 + K), 0)
    add("softcap_rows_kernel", (B if decode else 1) * cfg["vocab"] * 8, 0)
    return out


def _tofinex_twin_kernel_work(cfg, size, window, T, B, ctx, decode):
    W, H, G, d, ff, E, K, eff, sff = TOFINEX_SIZES[size]
    rows, layers = (B if decode else T), TOFINEX_LAYERS
    if decode:
        pairs, by = B * ctx, B * ctx * G * 2 * d * 2 + B * H * 2 * d * 2
        attn = "attn_decode_split_kernel"
    else:
        pairs = T * (T + 1) // 2
        by, attn = T * (H + G) * 2 * d * 2, "pt::attn_prefill_tc_kernel"
    return {attn: [layers * by, layers * pairs * H * 4.0 * d],
            "qkv_post_rows_kernel": [layers * rows * (H + 2 * G) * d * 6, 0.0],
            # residual read and written, a part's output in, the normalised row out
            "add_rmsnorm_vec_kernel": [(layers + 2) * rows * W * (4 + 8 + 2), 0.0],
            "combine_add_rmsnorm_vec_kernel": [(layers - 1) * rows * W * (4 * (K + 1) + 8 + 2), 0.0],
            "tc::gather_rows_kernel": [(layers - 1) * rows * W * 2 * (1 + K), 0.0]}


def run_tofinex(args):
    return _run_design(args, "tofinex", args.tofinex, 0, tofinex_config, tofinex_twin_config,
                       _tofinex_kernel_work, _tofinex_twin_kernel_work, "moe_twin", graph_prompts=True)


# --------------------------------------------------------------------------- #
# --bogetar: the Bogetar design beside the closest built-in model (Qwen2-MoE) at equal sizes
# --------------------------------------------------------------------------- #
BOGETAR_SIZES = {   # width, attention heads, key/value heads, head size, linear-attention heads, key size, value size,
                    # delta heads, delta key heads, experts, experts per token, expert width, expert groups (count, keep)
    "0.5b": (1024, 8, 2, 128, 8, 64, 128, 8, 4, 16, 2, 1024, (4, 2)),
    "a2.7b": (2048, 16, 4, 128, 16, 64, 128, 16, 8, 60, 4, 1408, (6, 3)),    # the expert sizes of Qwen1.5-MoE-A2.7B
}
BOGETAR_LAYERS = ("parallel", "delta", "parallel", "parallel", "delta", "parallel")


def bogetar_config(size, window, vocab):
    W, H, G, d, RH, rd, re, DH, DG, E, K, eff, groups = BOGETAR_SIZES[size]
    moe = {"kind": "moe", "expert": {"ff": eff, "limit": 7.0},
           "router": {"experts": E, "top": K, "groups": {"count": groups[0], "keep": groups[1]}}}
    parallel = {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "mask": {"size": window},
                         "rot": {"base": 500000.0, "dims": d // 2}, "scale": d ** -0.5},
                "right": {"heads": RH, "dim": rd, "vdim": re, "tau": 16.0, "decay_rank": 16},
                "left_scale": 0.6, "right_scale": 0.9}
    delta = {"heads": DH, "kv_heads": DG, "dim": d, "vdim": d, "conv": 4}
    layers = [{"type": t, "mixer": parallel if t == "parallel" else delta, "mlp": moe} for t in BOGETAR_LAYERS]
    return {"architecture": "Bogetar", "vocab": vocab, "width": W, "norm": {"eps": 1e-6, "groups": 2},
            "canon": {"taps": 4}, "layers": layers}


def bogetar_twin_config(size, window, vocab):
    """The closest built-in model: Qwen2-MoE with the same width, attention heads, window, experts and expert
    width, no shared expert, as many layers (all routed)."""
    W, H, G, d, RH, rd, re, DH, DG, E, K, eff, groups = BOGETAR_SIZES[size]
    return dict(A27B, vocab_size=vocab, hidden_size=W, intermediate_size=eff, num_hidden_layers=len(BOGETAR_LAYERS),
                num_attention_heads=H, num_key_value_heads=G, head_dim=d, num_experts=E, num_experts_per_tok=K,
                moe_intermediate_size=eff, shared_expert_intermediate_size=0, mlp_only_layers=[],
                norm_topk_prob=False, use_sliding_window=True, sliding_window=window, max_window_layers=0,
                max_position_embeddings=1 << 20)


def _bogetar_kernel_work(cfg, T, B, ctx, decode):
    """Algorithmic bytes and floating-point operations of the design's own kernels for one step over all layers
    (prefill of T tokens of one request, or a decode step of B requests at context ctx)."""
    rows, W, taps = (B if decode else T), cfg["width"], cfg["canon"]["taps"]
    out = {}

    def add(name, by, fl):
        a = out.setdefault(name, [0.0, 0.0])
        a[0] += by
        a[1] += fl

    def walk(H, G, d, e, form_columns):
        # rows in (q, k, v, and what the decays are made of), the prepared rows written and read, results out; the
        # state read and written once per request
        state = (B if decode else 1) * H * d * e * 4 * 2
        add("delta_scan_kernel", rows * (H * (3 * d + 4) + H * e * 2) * 4 + state, rows * H * d * e * 6.0)
        add("delta_prepare_kernel", rows * ((2 * G * d + form_columns) * 4 + H * (3 * d + 4) * 4), 0)
        add("gated_group_rmsnorm_kernel", rows * H * e * (4 + 4 + 2), 0)
    for L in cfg["layers"]:
        m = L["mixer"]
        if L["type"] == "delta":
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            ch = 2 * G * d + H * e
            walk(H, G, d, e, 2 * H)
            for name in ("causal_conv_silu_kernel", "causal_conv_silu_vec4_kernel"):
                add(name, rows * ch * 8, rows * ch * 8.0)
        else:
            a, r = m["left"], m["right"]
            H, G, d, e, win = a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["mask"]["size"]
            keys = min(ctx, win)
            pairs = B * keys if decode else sum(min(t + 1, win) for t in range(T))
            by = (B * keys * G * (d + e) * 2 + B * H * (d + e) * 2) if decode else T * (H + G) * (d + e) * 2
            for name in ("attn_mix_tc_kernel", "pt::attn_prefill_tc_kernel"):
                add(name, by, pairs * H * (2.0 * d + 2.0 * e))
            for name in ("rope_store_kernel", "rope_store_vec_kernel"):
                add(name, rows * (H * d + G * (d + e)) * 6, 0)
            add("sigmoid_gate_kernel", rows * H * e * (2 + 4 + 2), 0)
            walk(r["heads"], r["heads"], r["dim"], r["vdim"], r["heads"] * r["dim"])
        parts = 1 if L["mlp"] is None else 2
        # the residual's float32 row in, the normalised float32 row out; then the filter's taps and its rounded row
        add("group_rmsnorm_kernel", parts * rows * W * 8, 0)
        for name in ("causal_conv_silu_kernel", "causal_conv_silu_vec4_kernel"):
            add(name, parts * rows * W * (4 + 2), parts * rows * W * 2.0 * taps)
        # a part's float32 output in (two mixers' outputs, or the experts' rows), the residual read and written
        for name in ("out_norm_add_kernel", "out_norm_add_vec_kernel"):
            add(name, parts * rows * W * (4 + 8), 0)
            if L["type"] == "parallel":
                add(name, rows * W * 4, 0)
            if L["mlp"] is not None:
                add(name, rows * W * 4 * (L["mlp"]["router"]["top"] - 1), 0)
        if L["mlp"] is not None:
            add("tc::gather_rows_kernel", rows * W * 2 * (1 + L["mlp"]["router"]["top"]), 0)
    return out


def _bogetar_twin_kernel_work(cfg, size, window, T, B, ctx, decode):
    W, H, G, d = BOGETAR_SIZES[size][:4]
    K = BOGETAR_SIZES[size][10]
    rows, layers = (B if decode else T), len(BOGETAR_LAYERS)
    if decode:
        keys = min(ctx, window)
        pairs, by = B * keys, B * keys * G * 2 * d * 2 + B * H * 2 * d * 2
        attn = "attn_decode_split_kernel"
    else:
        pairs = sum(min(t + 1, window) for t in range(T))
        by, attn = T * (H + G) * 2 * d * 2, "pt::attn_prefill_tc_kernel"
    return {attn: [layers * by, layers * pairs * H * 4.0 * d],
            "qkv_post_rows_kernel": [layers * rows * (H + 2 * G) * d * 6, 0.0],
            "add_rmsnorm_vec_kernel": [(layers + 1) * rows * W * (4 + 8 + 2), 0.0],
            "combine_add_rmsnorm_vec_kernel": [layers * rows * W * (4 * (K + 1) + 8 + 2), 0.0],
            "tc::gather_rows_kernel": [layers * rows * W * 2 * (1 + K), 0.0]}


def run_bogetar(args):
    return _run_design(args, "bogetar", args.bogetar, args.bogetar_window, bogetar_config, bogetar_twin_config,
                       _bogetar_kernel_work, _bogetar_twin_kernel_work, "moe_twin", graph_prompts=True)


def run_reference(args):
    """The reference arm: Deyu-Kong/mini-infer itself, unmodified, built out of tree for sm_100 by
    ``baseline/build_reference.py`` and driven by ``baseline/reference_bench.cpp`` through its stock path
    (``ModelConfig::load`` -> ``TransformerModel::load_weights`` -> ``Scheduler::submit`` / ``Scheduler::step``) on a
    folder of the same layer sizes with random float16 weights (the reference computes in FP16 only) and
    seeded synthetic token ids.  Nothing of this repository's engine or kernels runs in that process; this
    function only writes the model folder, starts the program and reports what it measured."""
    import shutil
    import tempfile

    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    if args.gpus != 1:
        return unavailable("the reference engine runs on one GPU only")
    binary = os.path.join(ROOT, "baseline", "_ref", "reference_bench")
    if not os.path.exists(binary):
        source = os.environ.get("MINI_INFER_REFERENCE", "/root/reference")
        if not os.path.isfile(os.path.join(source, "CMakeLists.txt")):
            return unavailable("baseline/_ref/reference_bench is not built and no checkout of the reference is "
                               "at hand to build it from (python baseline/build_reference.py --source DIR)")
        p = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "build_reference.py"), "--source", source],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0 or not os.path.exists(binary):
            tail = " | ".join(p.stdout.strip().splitlines()[-3:])
            return unavailable(f"building the reference failed: {tail}")
    import torch
    from mini_infer_b200.weights.random_init import write_model_folder
    model_name, named = SIZES[args.sizes]
    cfg = dict(named)
    full_layers = named["num_hidden_layers"]
    if args.layers <= 0:
        args.layers = full_layers
    cfg["num_hidden_layers"] = args.layers
    cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], args.context)
    # the folder goes where there is room for it (about 29 GB at the headline sizes)
    best = max((d for d in (tempfile.gettempdir(), "/dev/shm") if os.path.isdir(d)),
               key=lambda d: shutil.disk_usage(d).free)
    folder = tempfile.mkdtemp(prefix="mini_infer_reference_", dir=best)
    try:
        t0 = time.time()
        write_model_folder(folder, cfg, seed=args.seed, dtype=torch.float16,
                           device="cuda:0" if torch.cuda.is_available() else "cpu")
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
        write_s = time.time() - t0
        clock = ClockSampler()
        clock.start()
        try:
            p = subprocess.run([binary, folder, str(args.batch), str(args.prompt_len), str(args.steps),
                                str(max(args.warmup, 3)), str(args.seed), str(args.reference_prefill_batch)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                               timeout=args.reference_timeout)
        except subprocess.TimeoutExpired:
            clock.stop()
            return unavailable(f"the reference did not finish within {args.reference_timeout} s")
        clocks = clock.stop()
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    result = None
    for line in p.stdout.splitlines():
        if line.startswith("RESULT "):
            result = json.loads(line[len("RESULT "):])
    if p.returncode != 0 or result is None:
        tail = " | ".join((p.stderr.strip() or p.stdout.strip()).splitlines()[-3:])
        return unavailable(f"the reference's program exited with {p.returncode}: {tail[:500]}")
    d = cfg["hidden_size"] // cfg["num_attention_heads"]
    out = {
        "metric": f"decode tok/s at batch {args.batch} ({model_name} sizes, {args.prompt_len}-token prompts)",
        "value": round(result["decode_tok_s"], 2), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(result["ms_per_step"], 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp16",
        "data": "synthetic: random-init weights, seeded uniform-random token ids", "impl": "reference",
        "config": {"model": f"{model_name} layer sizes (Qwen2MoeForCausalLM)", "global_batch": args.batch,
                   "seq_len": args.prompt_len, "context": args.context, "parallelism": "single GPU",
                   "layers": args.layers, "layers_of_named_config": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": d,
                   "experts": cfg["num_experts"], "top_k": cfg["num_experts_per_tok"],
                   "moe_intermediate": cfg["moe_intermediate_size"],
                   "shared_intermediate": cfg["shared_expert_intermediate_size"], "vocab": cfg["vocab_size"],
                   "page_size": 16, "l2": "every step reads GBs of weights (inputs larger than L2)",
                   "timing": "the reference scheduler's own clock (IterationStats.wall_ms) over iterations that "
                             "decode one token for every request and prefill nothing",
                   "reference_prefill_batch": result.get("prefill_batch")},
        # every iteration of the reference's scheduler uploads the token ids (int64) and reads the sampled
        # ids (int32) back, so its own clock is end to end already
        "e2e": {"value": round(result["decode_tok_s"], 2), "unit": "tok/s",
                "h2d_bytes_per_step": args.batch * 8, "d2h_bytes_per_step": args.batch * 4},
        "gpu_launches": None, "clocks": clocks,
        "reference": {"call_seconds": result["call_seconds"], "load_seconds": result["load_seconds"],
                      "write_seconds": round(write_s, 1), "generated": result["generated"]},
    }
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=0,
                    help="fewer layers than the named configuration has (same layer sizes) where memory or time "
                         "needs it; 0 = all of them")
    ap.add_argument("--sizes", default="a2.7b", choices=sorted(SIZES),
                    help="layer sizes: Qwen1.5-MoE-A2.7B (the headline configuration) or Qwen2-57B-A14B")
    ap.add_argument("--point-batches", default="1,64", help="batch sizes of the extra decode points")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-points", dest="points", action="store_false", help="skip decode at batch 1 and 64")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="run one workload and print a short line (used for profiling small cases)")
    ap.add_argument("--profiler-range", action="store_true",
                    help="wrap the timed region in cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    ap.add_argument("--eager", action="store_true", help="launch decode steps kernel by kernel, without CUDA graphs")
    ap.add_argument("--timeline", action="store_true",
                    help="print the kernels of one step as they run inside the engine (with --only decode or "
                         "--only prefill; --layers defaults to 4) instead of benchmarking")
    ap.add_argument("--serving", type=int, default=0,
                    help="instead of the benchmark line: this many requests of mixed prompt lengths through "
                         "LLM.generate as one continuous batch (throughput and time to first token)")
    ap.add_argument("--serving-new-tokens", type=int, default=128)
    ap.add_argument("--serving-prompt-min", type=int, default=100)
    ap.add_argument("--serving-prompt-max", type=int, default=2000)
    ap.add_argument("--serving-max-running", type=int, default=64)
    ap.add_argument("--vizalix", default="", metavar="SIZES",
                    help="instead of the default workload: the Vizalix design beside the closest built-in model at "
                         "these sizes (comma-separated, of " + ", ".join(VIZALIX_SIZES) + "), see run_vizalix")
    ap.add_argument("--vizalix-window", type=int, default=1024, help="attention window of the --vizalix models")
    ap.add_argument("--nipapel", default="", metavar="SIZES",
                    help="instead of the default workload: prefill and decode of the Nipapel design beside Qwen2-MoE at "
                         "these sizes (comma-separated, of " + ", ".join(NIPAPEL_SIZES) + "), see run_nipapel")
    ap.add_argument("--tofinex", default="", metavar="SIZES",
                    help="instead of the default workload: prefill and decode of the Tofinex design beside Qwen2-MoE at "
                         "these sizes (comma-separated, of " + ", ".join(TOFINEX_SIZES) + "), see run_tofinex")
    ap.add_argument("--nipapel-window", type=int, default=1024, help="attention window of the --nipapel models")
    ap.add_argument("--bogetar", default="", metavar="SIZES",
                    help="instead of the default workload: the Bogetar design beside Qwen2-MoE at "
                         "these sizes (comma-separated, of " + ", ".join(BOGETAR_SIZES) + "), see run_bogetar")
    ap.add_argument("--bogetar-window", type=int, default=1024, help="attention window of the --bogetar models")
    ap.add_argument("--reference-timeout", type=int, default=1500, help="seconds the reference's program may take")
    ap.add_argument("--reference-prefill-batch", type=int, default=1,
                    help="prompts the reference's scheduler prefills per iteration (its cuBLAS handles, one per "
                         "expert, and its per-expert activation buffers leave room for one 2,048-token prompt at a "
                         "time on 180 GB)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.timeline:
        return run_timeline(args)
    if args.serving > 0:
        return run_serving(args)
    if args.vizalix:
        return run_vizalix(args)
    if args.nipapel:
        return run_nipapel(args)
    if args.tofinex:
        return run_tofinex(args)
    if args.bogetar:
        return run_bogetar(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
