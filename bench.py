#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, Llama shapes with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--model llama31-8b|llama32-3b|llama2-7b] [--dtype bf16|fp16|fp32]
                    [--workload decode|serve|latent|hybrid|streams|delta] [--layers L] [--batch B] [--context S] [--trials N] [--size 2b|8b]

Prints ONE JSON line.

`--workload decode` (the default): `value` is decoded tokens per second at batch 8 with S cached
tokens per request (8192 for the 8B shape): the median of N trials (five by default), each of K
decode steps (forward pass of 8 single tokens over the paged cache, sampling included) timed with
CUDA events after W warm-up steps.  Trials of the different points alternate (batch 8, 1, 64,
then again), and every point reports median, minimum and maximum, the rule the reference sets for
its own numbers (docs/ARCHITECTURE.md:228).  `points` holds decode at batch 1 and 64 at the same
context, and the model's own decode workload (1024-token prompts and 256 new tokens for the 8B
shape, 4096-token prompts for the 3B shape): all 256 new tokens are timed.  `prefill` is a
2048-token prompt in one step; `roofline` is the decode step's bytes over its time against the
measured copy bandwidth; `e2e` is the headline point through `ferrum_b200.Engine.step()`: token
ids in from pinned host memory, sampled ids back to the host, every step.

`--workload serve`: continuous batching of 64 requests with prompts of 128 to 2048 tokens and
128 to 512 new tokens each, prompts cut into portions (`--chunk-size`), through `Engine`.
`value` is generated tokens per second over the whole run; the line also gives the time to the
first token (median and 95th percentile), preemptions, and what a step that cannot be replayed
from a CUDA graph costs the host.

`--workload latent`: the Ruperax design (latent attention in parallel gated blocks) at layer
sizes that resemble real models (`--size`), beside a Llama of equal size: prefill of a 2048-token
prompt, decode at batch 8 with 2048 cached tokens, and per kernel its time, bytes, flops and fraction
of the measured roofline.  `value` is the design's decode rate.

`--workload hybrid`: the same comparison for the Vikupel design (layers in turn: rotary attention with
unit-norm heads and turned values, a Mamba-2 mixer, windowed attention with a distance penalty and a
gate, a Mamba-2 mixer; parallel blocks with a per-layer token input) beside a Llama of equal width,
heads, feed-forward width and layers.

`--workload streams`: the same comparison for the Zavesun design (four residual streams around every
sublayer; layers in turn: windowed attention with distance slopes and a query temperature + dense
feed-forward, chunked rotary attention with biased, normed heads + eight experts of which a token takes
two, windowed + experts, chunked + dense; values blended with the first layer's; tied output matrix with
a soft cap) beside a Llama of equal width, heads, KV heads, layers and feed-forward width (the two chosen
experts together are as wide as the dense feed-forward).

`--workload delta`: the same comparison for the Pererax design (norms on the sublayers' results; layers in turn: a
pair of causal attention with a soft cap and a sink beside a matrix-memory recurrence, windowed attention whose
values are its keys, and two gated delta rules with a decay per key channel; every layer with eight clamped experts
plus two identity outputs, two per token, and a unit for every token) beside the closest of the other designs, a
Vikupel of equal width, heads, layers and active feed-forward width.

Weights are random N(0, 0.02); token ids are uniform random from a seed.  No L2 flush is needed
between steps: a step reads gigabytes of weights, far more than the 126 MB L2 holds.
"""
import argparse
import gc
import json
import os
import random
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA31_8B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 32, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256,
    "rope_theta": 500000.0, "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
}
# Two more shapes that the reference's workloads name, for `--model`.
LLAMA2_7B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 32, "num_attention_heads": 32,
    "num_key_value_heads": 32, "head_dim": 128, "intermediate_size": 11008, "vocab_size": 32000,
    "rope_theta": 10000.0, "max_position_embeddings": 4096, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
}
LLAMA32_3B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 3072, "num_hidden_layers": 28, "num_attention_heads": 24,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 8192, "vocab_size": 128256,
    "rope_theta": 500000.0, "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
}
# name -> (printed name, config, default context of the headline point, prompt length of the model's
# own decode workload or None)
MODELS = {"llama31-8b": ("Llama-3.1-8B", LLAMA31_8B, 8192, 1024), "llama2-7b": ("Llama-2-7B", LLAMA2_7B, 2048, None),
          "llama32-3b": ("Llama-3.2-3B", LLAMA32_3B, 4096, 4096)}
NEW_TOKENS = 256          # new tokens of the decode workloads
DTYPES = {"bf16": "bfloat16", "fp16": "float16", "fp32": "float32"}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        out = {k: float(d[k]) for k in ("hbm_gbs", "bf16_tflops") if k in d}
        if "bf16_tflops_sustained" in d:
            out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
        if "hbm_gbs" in out and "bf16_tflops" in out:
            out["source"] = "measured"
            return out
    except (OSError, ValueError, KeyError, TypeError):
        pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with NVML (read-only) while a region runs."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, period=0.1):
        self.period, self.samples, self.reasons, self.max_mhz = period, [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            idx = int(os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0] or 0)
            self._nv, self._h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self._nv.nvmlDeviceGetClockInfo(self._h, self._nv.NVML_CLOCK_SM))
                mask = self._nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def reference_arm():
    """The reference is a Rust workspace with no Python packaging and there is no Rust
    toolchain in this image, so it cannot be installed or run here."""
    print(json.dumps({"impl": "reference", "unavailable":
                      "JustinA988/ferrum is a CPU-only Rust workspace: pip reports 'neither setup.py nor "
                      "pyproject.toml found' and no cargo/rustc is installed, so it cannot be built offline"}))
    return 0


def layer_params(c):
    e, f = c["hidden_size"], c["intermediate_size"]
    q, kv = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    return e * q + 2 * e * kv + q * e + 3 * e * f


def spread(values, digits=1):
    """median, range and count of a point's trials."""
    return {"median": round(statistics.median(values), digits), "min": round(min(values), digits),
            "max": round(max(values), digits), "n": len(values)}


def shape_config(model_name, cfgd, L, full_layers, extra):
    out = {"model": f"{model_name} shape, random weights N(0,0.02)", "layers": L, "layers_full_model": full_layers,
           "hidden": cfgd["hidden_size"], "heads": cfgd["num_attention_heads"], "kv_heads": cfgd["num_key_value_heads"],
           "head_dim": cfgd["head_dim"], "intermediate": cfgd["intermediate_size"], "vocab": cfgd["vocab_size"]}
    out.update(extra)
    assert len(out) <= 20
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in config)")
    ap.add_argument("--model", default="llama31-8b", choices=sorted(MODELS), help="layer sizes (random weights)")
    ap.add_argument("--dtype", default="bf16", choices=sorted(DTYPES), help="compute dtype; fp32 is the true 32-bit path")
    ap.add_argument("--workload", default="decode", choices=["decode", "serve", "latent", "hybrid", "streams", "delta"])
    ap.add_argument("--size", default="2b", choices=sorted(LATENT_SIZES), help="latent, hybrid, streams, delta: the layer sizes to compare at")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=None,
                    help="cached tokens per request of the headline point (default 8192 for llama31-8b, 4096 for "
                         "llama32-3b, 2048 for llama2-7b and for fp32: what lets the batch-64 point fit the memory)")
    ap.add_argument("--trials", type=int, default=5, help="timed regions per point; median and range are reported")
    ap.add_argument("--chunk-size", type=int, default=512, help="serve: the longest prompt portion of a step")
    ap.add_argument("--requests", type=int, default=64, help="serve: number of requests")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-prefill", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus %d is not supported" % args.gpus)
        return 2
    if args.workload == "serve":
        return serve(args)
    if args.workload == "latent":
        return latent(args)
    if args.workload == "hybrid":
        return latent(args, design="vikupel")
    if args.workload == "streams":
        return latent(args, design="zavesun")
    if args.workload == "delta":
        return latent(args, design="pererax")
    return decode(args)


def build_model(args, max_positions):
    import torch
    from ferrum_b200.config import registry
    from ferrum_b200.engine.api import parse_dtype
    from ferrum_b200.weights import init_random
    model_name, shape, _, _ = MODELS[args.model]
    cfgd = dict(shape)
    full_layers = cfgd["num_hidden_layers"]
    if args.layers:
        cfgd["num_hidden_layers"] = args.layers
    arch = registry.lookup(cfgd["architectures"][0])
    cfg = arch.read_config(cfgd)
    td = parse_dtype(DTYPES[args.dtype])
    torch.manual_seed(0)
    model = arch.build(cfg, td, "cuda", max_positions=max_positions)
    init_random(model, 0, "cuda")
    return model, cfg, cfgd, td, model_name, full_layers


# ---------------------------------------------------------------------------------- decode workload
def decode(args):
    import torch
    from ferrum_b200.cache import CacheStorage
    from ferrum_b200.engine import ModelRunner, StepEntry
    from ferrum_b200.engine.api import Engine
    from ferrum_b200.ops import lib as ops

    W, K, N_TRIALS = max(3, args.warmup), max(1, args.steps), max(1, args.trials)
    pk = peaks()
    _, _, default_ctx, prompt_len = MODELS[args.model]
    if args.context is None:
        args.context = min(default_ctx, 2048) if args.dtype == "fp32" else default_ctx
    ctx_len, B = args.context, args.batch
    esize = 4 if args.dtype == "fp32" else 2
    page = 16
    max_len = max(ctx_len, (prompt_len or 0) + NEW_TOKENS) + W + K + 128 + 4 * B
    model, cfg, cfgd, td, model_name, full_layers = build_model(args, max_len)
    L = cfgd["num_hidden_layers"]
    gen = torch.Generator().manual_seed(0)

    def tokens(n):
        return torch.randint(0, cfg.n_vocab, (n,), generator=gen).tolist()

    tied = bool(cfgd.get("tie_word_embeddings"))
    weight_bytes = esize * (L * layer_params(cfgd) + cfgd["vocab_size"] * cfgd["hidden_size"]) + 4 * (2 * L + 1) * cfgd["hidden_size"]
    kv_per_token = 2 * cfgd["num_key_value_heads"] * cfgd["head_dim"] * esize * L

    # One cache and one runner serve every point: requests are opened at the point's context and
    # closed after its trial, so trials of different points can alternate.
    max_b = B if args.skip_points else max(B, 64)
    cache = CacheStorage(model, td, "cuda", page_size=page, max_tokens=max_b * (max_len + page), max_requests=max_b,
                         max_model_len=max_len)
    for p in cache.pools:
        p.normal_(0.0, 0.02)                       # contents of a cache that earlier steps left
    runner = ModelRunner(model, cache, max_batch_tokens=2048, max_batch_requests=max_b)
    mgr = cache.manager
    ids = torch.empty(max_b, dtype=torch.int32, device="cuda")

    def decode_trial(batch, start, steps, warm):
        """`steps` timed decode steps of `batch` requests that hold `start` tokens each when timing
        begins (the warm-up steps come before, at shorter contexts).  (tok/s, ms per step, launches)"""
        slots = [cache.open() for _ in range(batch)]
        first = start - warm
        for s in slots:
            mgr.grow(s, first - 1)
            mgr.commit(s, first - 1)

        def one(i):
            entries = [StepEntry(s, first - 1 + i, [t], [0]) for s, t in zip(slots, tokens(batch))]
            logits = runner.step(entries, check=False)
            ops.sample(logits, batch, ids, runner.ctx.err)

        for i in range(warm):
            one(i)
        torch.cuda.synchronize()
        l0 = ops.launches
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for i in range(steps):
            one(warm + i)
        ev1.record()
        torch.cuda.synchronize()
        runner.check_device_errors()
        ms = ev0.elapsed_time(ev1) / steps
        launches = ops.launches - l0
        for s in slots:
            cache.close(s)
        return batch / ms * 1e3, ms, launches

    # (name, batch, context at the first timed step, timed steps)
    plan = [(f"decode_b{B}", B, ctx_len, K)]
    if not args.skip_points:
        plan += [(f"decode_b{b}", b, ctx_len, max(4, K // 2)) for b in (1, 64) if b != B]
        if prompt_len:
            plan += [(f"decode_b{b}_prompt{prompt_len}_new{NEW_TOKENS}", b, prompt_len, NEW_TOKENS) for b in (1, 8, 64)]
    results = {name: [] for name, *_ in plan}
    ms_main, launches = [], 0
    with ClockSampler() as clk:
        for trial in range(N_TRIALS):
            for name, b, start, steps in plan:
                r, ms, n = decode_trial(b, start, steps, W)
                results[name].append(r)
                if name == plan[0][0]:
                    ms_main.append(ms)
                    launches = n
    clocks = clk.summary()
    value = statistics.median(results[plan[0][0]])
    ms_step = statistics.median(ms_main)
    step_bytes = weight_bytes + B * cfgd["hidden_size"] * esize + B * ctx_len * kv_per_token
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"]}
    points, trials = {}, {}
    for name, b, start, steps in plan:
        trials[name] = spread(results[name])
        if name != plan[0][0]:
            points[name] = trials[name]["median"]
            # every point against the copy peak: weights once, the cache of its requests (mean context)
            mean_ctx = start + (steps - 1) / 2
            bytes_ = weight_bytes + b * mean_ctx * kv_per_token
            trials[name]["hbm_frac"] = round(bytes_ * trials[name]["median"] / b / 1e9 / pk["hbm_gbs"], 4)

    # ------------------------------------------------------------ prefill of 2048 tokens
    prefill = None
    if not args.skip_prefill:
        T = 2048
        times = []
        for it in range(W + N_TRIALS):
            slot = cache.open()
            toks = tokens(T)
            torch.cuda.synchronize()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            runner.step([StepEntry(slot, 0, toks, [T - 1])], check=False)
            ev1.record()
            torch.cuda.synchronize()
            if it >= W:
                times.append(ev0.elapsed_time(ev1))
            cache.close(slot)
        runner.check_device_errors()
        ms = statistics.median(times)
        hq, d = cfgd["num_attention_heads"], cfgd["head_dim"]
        flops = 2.0 * L * layer_params(cfgd) * T + 2.0 * cfgd["vocab_size"] * cfgd["hidden_size"] + L * 4.0 * hq * d * T * T / 2
        if args.dtype == "fp32":     # the CUDA cores' own peak: SMs x 128 lanes x 2 flops x the maximum clock
            peak, of = ops.sm_count() * 128 * 2 * (clocks["sm_max_mhz"] or 1965) * 1e6, "nominal ffma"
        else:
            peak, of = pk["bf16_tflops"] * 1e12, pk["source"]
        prefill = {"value": round(T / ms * 1e3, 1), "tokens": T, "ms": round(ms, 3), "ms_min": round(min(times), 3),
                   "ms_max": round(max(times), 3), "frac": round(flops / (ms * 1e-3) / peak, 4), "of": of}
    del runner, cache
    torch.cuda.empty_cache()

    # ------------------------------------------------------------ end to end through the Engine
    e2e = None
    if not args.skip_e2e:
        eng = Engine(model=model, page_size=page, num_pages=(B * (max_len + page)) // page, max_batch_tokens=8192,
                     max_batch_seqs=B, max_model_len=max_len)
        for _ in range(B):
            eng.submit(tokens(ctx_len - 1), W + K + 80 + 4 * B)
        started = set()
        while len(started) < B:                        # prompts, untimed; ends with every request decoding
            started.update(ev.id for ev in eng.step() if ev.kind == "token")
        # The prompts have just run at the power cap; the first dozen decode steps after them are
        # up to 10 % slow while the clocks come back.  They are part of the warm-up.
        e2e_warm = W + 16
        for _ in range(e2e_warm):
            eng.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        got = 0
        for _ in range(K):
            got += sum(1 for ev in eng.step() if ev.kind == "token")
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        assert got == B * K, (got, B * K)
        e2e = {"value": round(got / dt, 1), "unit": "tok/s", "h2d_bytes_per_step": int(eng.runner.ctx.h2d_bytes),
               "d2h_bytes_per_step": int(eng.sampler.d2h_bytes), "ms_per_step": round(dt / K * 1e3, 3),
               "warmup": e2e_warm}

    line = {
        "metric": f"decode tok/s ({model_name} {args.dtype}, batch {B}, context {ctx_len})", "value": round(value, 1),
        "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic", "impl": "ours",
        "config": shape_config(model_name, cfgd, L, full_layers, {
            "global_batch": B, "seq_len": ctx_len, "page_size": page, "prefill_tokens": 2048, "parallelism": "single GPU",
            "trials": f"{N_TRIALS} alternating trials per point, median reported",
            "l2": f"inputs larger than L2 ({weight_bytes / 1e9:.0f} GB of weights per step)",
            "sampling": "greedy on device, inside the step", "tied_output": tied}),
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "prefill": prefill, "roofline": roofline,
        "points": points, "trials": trials,
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------- serving workload
def serve(args):
    """Continuous batching through the Python entry point, the reference's fourth configuration:
    64 requests, prompt lengths uniform in [128, 2048], 128 to 512 new tokens, chunked prefill."""
    import torch
    from ferrum_b200.engine.api import Engine
    from ferrum_b200.ops import lib as ops

    pk = peaks()
    n_req, chunk = args.requests, args.chunk_size
    max_len = 2048 + 512 + 16
    model, cfg, cfgd, td, model_name, full_layers = build_model(args, max_len)
    L = cfgd["num_hidden_layers"]
    rng = random.Random(0)
    reqs = [(rng.randint(128, 2048), rng.randint(128, 512)) for _ in range(n_req)]
    page = 16
    runs = []
    clk = ClockSampler()
    with clk:
        for rep in range(2):                              # the first run compiles nothing but captures the graphs
            eng = Engine(model=model, page_size=page, num_pages=(n_req * max_len) // page, max_batch_tokens=2048,
                         max_batch_seqs=n_req, chunk_size=chunk, max_model_len=max_len)
            gen = torch.Generator().manual_seed(1)
            launch_ms = []
            inner = eng._launch

            def timed_launch(plan, ahead_of_commit=False, inner=inner, launch_ms=launch_ms):
                replays = eng.runner.graph_replays
                t = time.perf_counter()
                out = inner(plan, ahead_of_commit=ahead_of_commit)
                if eng.runner.graph_replays == replays:      # launched kernel by kernel: what the host spends on it
                    launch_ms.append((time.perf_counter() - t) * 1e3)
                return out

            eng._launch = timed_launch
            ids = [eng.submit(torch.randint(0, cfg.n_vocab, (n,), generator=gen).tolist(), new) for n, new in reqs]
            torch.cuda.synchronize()
            l0 = ops.launches
            t0 = time.perf_counter()
            first, done, generated, steps = {}, 0, 0, 0
            while done < n_req:
                events = eng.step()
                now = time.perf_counter()
                steps += 1
                for ev in events:
                    if ev.kind == "token":
                        generated += 1
                        first.setdefault(ev.id, now - t0)
                    else:
                        done += 1
            while eng.step():
                pass
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            st = eng.stats()
            ttft = sorted(first[i] for i in ids)
            runs.append({"seconds": round(dt, 3), "generated_tok_s": round(generated / dt, 1),
                         "total_tok_s": round((generated + st["prompt_tokens"]) / dt, 1), "steps": steps,
                         "generated": generated, "prompt_tokens": int(st["prompt_tokens"]),
                         "ttft_ms_median": round(statistics.median(ttft) * 1e3, 1),
                         "ttft_ms_p95": round(ttft[min(len(ttft) - 1, int(0.95 * len(ttft)))] * 1e3, 1),
                         "preemptions": int(st["preemptions"]), "graph_replays": int(eng.runner.graph_replays),
                         "non_graph_steps": len(launch_ms),
                         "host_ms_per_non_graph_step": round(statistics.median(launch_ms), 3) if launch_ms else None,
                         "gpu_launches": int(ops.launches - l0)})
            eng._launch = None            # (the timing wrapper holds the engine: break the cycle so that its cache is freed)
            del eng, inner, timed_launch
            gc.collect()
            torch.cuda.empty_cache()
    best = runs[-1]
    line = {
        "metric": f"generated tok/s ({model_name} {args.dtype}, {n_req} requests, prompts U[128,2048], 128-512 new tokens, "
                  f"continuous batching, portions of {chunk})",
        "value": best["generated_tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": best["steps"], "warmup": runs[0]["steps"],
        "ms_per_step": round(best["seconds"] / best["steps"] * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": args.dtype, "data": "synthetic", "impl": "ours",
        "config": shape_config(model_name, cfgd, L, full_layers, {
            "global_batch": n_req, "seq_len": 2560, "page_size": page, "chunk_size": chunk, "max_batch_tokens": 2048,
            "parallelism": "single GPU", "l2": "inputs larger than L2 (the weights are read every step)",
            "sampling": "greedy on device, inside the step",
            "timing": "host clock around the whole run, after one identical warm-up run"}),
        "clocks": clk.summary(), "serve": best, "warmup_run": runs[0], "gpu_launches": best["gpu_launches"],
        "e2e": {"value": best["generated_tok_s"], "unit": "tok/s", "note": "the workload itself runs through Engine.step()"},
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------- latent attention beside Llama
# Layer sizes that resemble real models; the Llama beside each has the same width, heads, head size,
# feed-forward width, layers and vocabulary (a quarter as many KV heads as heads).
LATENT_SIZES = {
    "2b": dict(width=2048, heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=768, ff=5632),
    "8b": dict(width=4096, heads=32, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=1536, ff=14336),
}


def latent_configs(size, layers, vocab=32000, window=4096, groups=8):
    s = LATENT_SIZES[size]
    mixer = {"heads": s["heads"], "dim": s["dim"], "rot_dim": s["rot_dim"], "vdim": s["vdim"], "kv_rank": s["kv_rank"],
             "q_rank": s["q_rank"], "scale": (s["dim"] + s["rot_dim"]) ** -0.5, "mask": {"size": window},
             "rot": {"base": 10000.0, "dims": s["rot_dim"]}}
    ours = {"architecture": "Ruperax", "vocab": vocab, "width": s["width"], "max_positions": 4096, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6, "groups": groups},
            "layers": [{"type": "latent_attention", "mixer": dict(mixer), "mlp": {"kind": "dense", "ff": s["ff"]}}
                       for _ in range(layers)]}
    llama = {"architectures": ["LlamaForCausalLM"], "hidden_size": s["width"], "num_hidden_layers": layers,
             "num_attention_heads": s["heads"], "num_key_value_heads": max(1, s["heads"] // 4), "head_dim": 128,
             "intermediate_size": s["ff"], "vocab_size": vocab, "rope_theta": 10000.0, "max_position_embeddings": 4096,
             "rms_norm_eps": 1e-6, "tie_word_embeddings": False}
    return ours, llama


# Vikupel at the same two widths: attention heads of 128 (a quarter as many KV heads), the recurrent
# mixer twice as wide as the model with heads of 64 and a state of 128, a per-layer token input of 256.
HYBRID_SIZES = {
    "2b": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, ssm_heads=64, ssm_vdim=64, state=128, ff=5632, side=256),
    "8b": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, ssm_heads=128, ssm_vdim=64, state=128, ff=14336, side=256),
}


def hybrid_configs(size, layers, vocab=32000, window=1024):
    """Layers in turn: rotary attention, recurrent, windowed attention, recurrent; and the Llama beside it."""
    s = HYBRID_SIZES[size]
    att = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"], "scale": s["dim"] ** -0.5}
    kinds = [{"type": "attention_2", "mixer": dict(att, rot={"base": 500000.0, "dims": s["dim"], "scaling": {
                  "factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}})},
             {"type": "mamba2", "mixer": {"heads": s["ssm_heads"], "vdim": s["ssm_vdim"], "state": s["state"], "groups": 1,
                                          "norm_groups": 1, "conv": 4}},
             {"type": "attention", "mixer": dict(att, mask={"size": window})},
             {"type": "mamba2", "mixer": {"heads": s["ssm_heads"], "vdim": s["ssm_vdim"], "state": s["state"], "groups": 1,
                                          "norm_groups": 1, "conv": 4}}]
    ours = {"architecture": "Vikupel", "vocab": vocab, "width": s["width"], "norm": {"eps": 1e-6}, "residual_mult": 0.7,
            "token_side": {"dim": s["side"]},
            "layers": [dict(kinds[i % 4], mlp={"kind": "dense", "ff": s["ff"]}) for i in range(layers)]}
    llama = {"architectures": ["LlamaForCausalLM"], "hidden_size": s["width"], "num_hidden_layers": layers,
             "num_attention_heads": s["heads"], "num_key_value_heads": s["kv_heads"], "head_dim": 128,
             "intermediate_size": s["ff"], "vocab_size": vocab, "rope_theta": 500000.0, "max_position_embeddings": 4096,
             "rms_norm_eps": 1e-6, "tie_word_embeddings": False}
    return ours, llama


# Zavesun at the same two widths: heads of 128 (a quarter as many KV heads), four residual streams, eight experts
# half as wide as the dense feed-forward, two per token.
STREAM_SIZES = {
    "2b": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, ff=5632, experts=8, top=2, expert_ff=2816, streams=4),
    "8b": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, ff=14336, experts=8, top=2, expert_ff=7168, streams=4),
}


def stream_configs(size, layers, vocab=32000, window=1024):
    """Layers in turn: windowed + dense, chunked + experts, windowed + experts, chunked + dense; and the Llama beside it."""
    s = STREAM_SIZES[size]
    att = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"], "scale": s["dim"] ** -0.5,
           "mask": {"size": window}, "v_mix": True}
    windowed = {"type": "attention", "mixer": dict(att, q_temp={"coef": 0.25, "every": 256})}
    chunked = {"type": "attention_2", "mixer": dict(att, rot={"base": 10000.0, "dims": s["dim"] // 2, "scaling": {"factor": 4.0}})}
    dense = {"kind": "dense", "ff": s["ff"]}
    routed = {"kind": "moe", "expert": {"ff": s["expert_ff"]}, "router": {"experts": s["experts"], "top": s["top"]}}
    kinds = [dict(windowed, mlp=dense), dict(chunked, mlp=routed), dict(windowed, mlp=routed), dict(chunked, mlp=dense)]
    ours = {"architecture": "Zavesun", "vocab": vocab, "width": s["width"], "norm": {"eps": 1e-6}, "streams": s["streams"],
            "logit_softcap": 30.0, "layers": [kinds[i % 4] for i in range(layers)]}
    llama = {"architectures": ["LlamaForCausalLM"], "hidden_size": s["width"], "num_hidden_layers": layers,
             "num_attention_heads": s["heads"], "num_key_value_heads": s["kv_heads"], "head_dim": 128,
             "intermediate_size": s["ff"], "vocab_size": vocab, "rope_theta": 10000.0, "max_position_embeddings": 4096,
             "rms_norm_eps": 1e-6, "tie_word_embeddings": False}
    return ours, llama


# Pererax at the same two widths: attention heads of 128 (a quarter as many KV heads), recurrent heads with a 128 x 128
# memory each, eight experts a quarter as wide as the dense feed-forward plus two identity outputs, two per token, and
# a unit for every token half as wide as the dense feed-forward (so a token's active width equals the dense one).
DELTA_SIZES = {
    "2b": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, memory_heads=16, rank=128, experts=8, identity=2, top=2,
               expert_ff=1408, shared_ff=2816),
    "8b": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, memory_heads=32, rank=128, experts=8, identity=2, top=2,
               expert_ff=3584, shared_ff=7168),
}


def delta_configs(size, layers, vocab=32000, window=1024):
    """Layers in turn: the pair (sink attention beside matrix memory), windowed attention with its keys as values,
    delta rule, delta rule; and the Vikupel of equal size beside it."""
    s = DELTA_SIZES[size]
    att = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"], "scale": s["dim"] ** -0.5,
           "rot": {"base": 500000.0, "dims": s["dim"]}}
    memory = {"heads": s["memory_heads"], "dim": s["dim"], "vdim": s["vdim"], "gate_cap": 15.0}
    delta = {"heads": s["memory_heads"], "kv_heads": s["memory_heads"], "dim": s["dim"], "vdim": s["vdim"], "conv": 4,
             "decay_rank": s["rank"], "gate_rank": s["rank"]}
    mlp = {"kind": "moe", "expert": {"ff": s["expert_ff"], "limit": 7.0}, "shared": {"ff": s["shared_ff"], "limit": 7.0},
           "router": {"experts": s["experts"], "identity": s["identity"], "top": s["top"], "scale": 2.5}}
    kinds = [{"type": "parallel", "mixer": {"left": dict(att, softcap=50.0), "right": memory}},
             {"type": "attention", "mixer": dict(att, mask={"size": window})},
             {"type": "channel_delta", "mixer": delta}, {"type": "channel_delta", "mixer": delta}]
    ours = {"architecture": "Pererax", "vocab": vocab, "width": s["width"], "norm": {"eps": 1e-6},
            "layers": [dict(kinds[i % 4], mlp=mlp) for i in range(layers)]}
    return ours, hybrid_configs(size, layers, vocab, window)[0]


# design -> (title, configs of the design and of the model beside it, sizes, window, what stands beside it)
DESIGNS = {"ruperax": ("Ruperax", latent_configs, LATENT_SIZES, 4096, "llama"), "vikupel": ("Vikupel", hybrid_configs, HYBRID_SIZES, 1024, "llama"),
           "zavesun": ("Zavesun", stream_configs, STREAM_SIZES, 1024, "llama"),
           "pererax": ("Pererax", delta_configs, DELTA_SIZES, 1024, "vikupel")}


def latent(args, design="ruperax"):
    """Prefill (one 2048-token prompt in one step) and decode (batch 8 at 2048 cached tokens) of the
    Ruperax design at real layer sizes beside a Llama of equal size, random weights, and per kernel
    the time of one such step with its bytes, flops and fraction of the measured roofline (from
    a profiled pass that launches kernel by kernel)."""
    import torch
    from ferrum_b200.cache import CacheStorage
    from ferrum_b200.config import registry
    from ferrum_b200.engine import ModelRunner, StepEntry
    from ferrum_b200.engine.api import parse_dtype
    from ferrum_b200.ops import lib as ops
    from ferrum_b200.weights import init_random

    W, K, N_TRIALS = max(3, args.warmup), max(1, args.steps), max(1, args.trials)
    L = args.layers or 4
    B, ctx_len, T = args.batch, args.context or 2048, 2048
    td = parse_dtype(DTYPES[args.dtype])
    pk = peaks()
    page = 16
    max_len = max(ctx_len, T) + W + K + 64
    gen = torch.Generator().manual_seed(0)
    out = {}
    with ClockSampler() as clk:
        title, make_configs, all_sizes, window, beside = DESIGNS[design]
        configs = make_configs(args.size, L)
        for name, cfgd in zip((design, beside), configs):
            arch = registry.lookup(registry.architecture_name(cfgd))
            cfg = arch.read_config(cfgd)
            model = arch.build(cfg, td, "cuda", max_positions=max_len)
            init_random(model, 0, "cuda")
            cache = CacheStorage(model, td, "cuda", page_size=page, max_tokens=B * (max_len + page), max_requests=B,
                                 max_model_len=max_len)
            for p in cache.pools:
                p.normal_(0.0, 0.5)
            runner = ModelRunner(model, cache, max_batch_tokens=T, max_batch_requests=B)
            mgr = cache.manager
            ids = torch.empty(B, dtype=torch.int32, device="cuda")

            def tokens(n):
                return torch.randint(0, cfg.n_vocab, (n,), generator=gen).tolist()

            def prefill_once():
                slot = cache.open()
                toks = tokens(T)
                torch.cuda.synchronize()
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record()
                runner.step([StepEntry(slot, 0, toks, [T - 1])], check=False)
                ev1.record()
                torch.cuda.synchronize()
                cache.close(slot)
                return ev0.elapsed_time(ev1)

            def decode_run(steps, warm):
                slots = [cache.open() for _ in range(B)]
                first = ctx_len - warm
                for s in slots:
                    mgr.grow(s, first - 1)
                    mgr.commit(s, first - 1)
                l0 = 0
                for i in range(warm + steps):
                    if i == warm:
                        torch.cuda.synchronize()
                        l0 = ops.launches
                        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        ev0.record()
                    entries = [StepEntry(s, first - 1 + i, [t], [0]) for s, t in zip(slots, tokens(B))]
                    ops.sample(runner.step(entries, check=False), B, ids, runner.ctx.err)
                ev1.record()
                torch.cuda.synchronize()
                n = ops.launches - l0
                for s in slots:
                    cache.close(s)
                return ev0.elapsed_time(ev1) / steps, n

            pre = [prefill_once() for _ in range(W + N_TRIALS)][W:]
            dec = [decode_run(K, W) for _ in range(N_TRIALS)]
            runner.check_device_errors()
            # per kernel: one prompt step and four decode steps launched kernel by kernel
            runner.use_graphs = False
            kernels = {}
            for what, fn in (("prefill", prefill_once), ("decode", lambda: decode_run(4, 1))):
                fn()
                ops.profile_begin()
                fn()
                rows = ops.profile_report(pk)
                steps = 1 if what == "prefill" else 5
                kernels[what] = [{"kernel": r["kernel"], "launches_per_step": round(r["launches"] / steps, 1),
                                  "us_per_step": round(r["ms"] * 1e3 / steps, 1), "GBps": r.get("GBps"), "TFLOPs": r.get("TFLOPs"),
                                  "frac": r.get("frac_of_roofline")} for r in rows]
            ms_p, ms_d = statistics.median(pre), statistics.median([d[0] for d in dec])
            out[name] = {"prefill_tok_s": round(T / ms_p * 1e3, 1), "prefill_ms": round(ms_p, 3),
                         "decode_tok_s": round(B / ms_d * 1e3, 1), "decode_ms_per_step": round(ms_d, 4),
                         "decode_launches_per_step": dec[0][1] // K, "kernels": kernels,
                         "cache_bytes_per_token": CacheStorage.bytes_per_token_of(model, td)}
            del runner, cache, model
            gc.collect()
            torch.cuda.empty_cache()
    ours = out[design]
    sizes = all_sizes[args.size]
    line = {"metric": f"decode tok/s ({title} {args.size} layer sizes, {args.dtype}, batch {B}, context {ctx_len})",
            "value": ours["decode_tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W,
            "ms_per_step": ours["decode_ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": args.dtype, "data": "synthetic", "impl": "ours",
            "config": dict(sizes, model=f"{title}, {args.size} layer sizes, random weights", layers=L,
                           global_batch=B, seq_len=ctx_len, prefill_tokens=T, window=window,
                           vocab=32000, page_size=page,
                           parallelism="single GPU", l2="weights of a step exceed the L2 at these sizes"),
            "clocks": clk.summary(), "gpu_launches": int(ours["decode_launches_per_step"] * K), "peaks": pk,
            design: ours, beside + "_equal_size": out[beside]}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
