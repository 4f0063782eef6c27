"""Decode and prefill throughput of the engine on one B200, Qwen2.5-7B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 with contexts
that end at 4,096 tokens, timed on the device with CUDA events over exactly K decode
steps of the engine's step function (bfloat16, seeded random weights of the full
28-layer shape, uniform random token ids).  ``e2e`` is the same through the public
``LLMEngine.step()`` loop: host token ids in (one pinned host-to-device copy per step)
and sampled tokens out (one device-to-host copy per step).  ``prefill`` is one
2,048-token prompt in one step; ``points`` holds decode at batch 1 and 64; ``roofline``
divides the bytes a decode step has to read (every weight once, the cache of the live
requests) by its time and by the measured copy bandwidth.

A decode step reads far more than the 126 MB of L2 (14 GB of weights), so consecutive
timed steps never find their inputs cached: "inputs larger than L2" in ``config``.

The same line carries, under ``points``, every other measurement of the engine: decode and
prefill of the true 32-bit path, prefill at 128 / 256 / 512 tokens, a mixed step (32 decoding
rows beside a 512-token prompt portion), the hot kernels alone as fractions of the measured
peaks, continuous batching of 256 requests at the 0.5B shape and chunked prefill beside decode
at the 32B shape (the last three models are built in child processes of their own, one after
the other, once this process has freed the GPU; ``--no-extras`` leaves them out).

``--impl reference`` runs the unmodified reference from ``baseline/_ref`` through its own
``LLMEngine`` for the same metric and shape, or prints why it cannot.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# Layer sizes of the Qwen2.5-7B shape (third configuration of the baseline description).
SHAPE_7B = dict(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
                num_attention_heads=28, num_key_value_heads=4, head_dim=128,
                max_position_embeddings=32768, rms_norm_eps=1e-6, rope_theta=1_000_000.0,
                tie_word_embeddings=False, attention_bias=True, eos_token_id=151645)
CONTEXT = 4096
PREFILL_TOKENS = 2048
PAGE_SIZE = 16
# The reference publishes no B200 number for this metric; its A100 fp16 figure for the
# same shape at batch 8 (10.64 ms per step) is quoted for context only.
A100_FP16_B8_TOK_S = 752.0

CLOCK_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
               "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
               "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def measured_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        d = json.loads(path.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    def __init__(self) -> None:
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={CLOCK_QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", "0"], stdout=self.file, stderr=subprocess.DEVNULL)
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

    def summary(self) -> dict:
        self.file.flush()
        rows = [line.split(",") for line in Path(self.file.name).read_text().splitlines() if line.strip()]
        os.unlink(self.file.name)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, cell in zip(names, r[5:9]):
                if cell.strip().lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        busy = [s for s in sm if s >= 0.5 * max(sm)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def model_bytes_and_flops(cfg, layers: int) -> dict:
    h, i, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    per_layer = h * (q + 2 * kv) + (q + 2 * kv) + q * h + 3 * h * i + 2 * h
    return {"layer_params": per_layer, "weight_bytes": 2 * (layers * per_layer + v * h + h),
            "kv_bytes_per_token": 2 * layers * 2 * kv,
            "linear_flops_per_token": 2 * layers * (h * (q + 2 * kv) + q * h + 3 * h * i),
            "attn_flops_causal": lambda t: layers * 4 * q * t * t / 2, "head_flops": 2 * v * h}


def run_ours(args) -> dict:
    import torch

    from emberserve_b200 import kernels as K
    from emberserve_b200.config.engine import EngineConfig
    from emberserve_b200.config.model import Qwen2Config
    from emberserve_b200.engine.llm_engine import LLMEngine
    from emberserve_b200.engine.runner import ModelRunner, StepRow
    from emberserve_b200.sampling.params import SamplingParams

    assert torch.cuda.is_available(), "bench.py needs a CUDA GPU"
    peaks = measured_peaks()
    shape = dict({"7b": SHAPE_7B, "0.5b": SHAPE_05B, "32b": SHAPE_32B}[args.model_shape])
    full_layers = shape["num_hidden_layers"]
    shape["num_hidden_layers"] = args.layers or full_layers
    cfg = Qwen2Config.from_dict(dict(shape, architectures=["Qwen2ForCausalLM"], model_type="qwen2"))
    layers = cfg.num_hidden_layers
    K.library()
    torch.manual_seed(0)
    max_b = max(64, args.batch)
    ctx_cap = CONTEXT
    if args.only == "decode":  # a single phase at another context: size the pool and the graphs for it
        max_b, ctx_cap = args.batch, max(CONTEXT, args.decode_context)
    ptoks = args.prefill_tokens if args.only == "prefill" else PREFILL_TOKENS
    if args.only == "prefill":
        max_b = 1
    pages = max_b * (ctx_cap // PAGE_SIZE + 1) + 2 * (ptoks // PAGE_SIZE) + 64
    dtype = torch.float32 if args.dtype == "float32" else torch.bfloat16
    runner = ModelRunner.from_random(cfg, seed=0, dtype=dtype, device="cuda:0",
                                     page_size=PAGE_SIZE, num_pages=pages,
                                     tiled_weight_copies=False if args.no_tiled_weights else None)
    if not args.no_graphs:
        runner.enable_graphs(ctx_cap + 64, max_b)
    for t in runner.storage.tensors:  # keys and values of the "earlier" tokens: random, not zero
        t.normal_(0, 1)
    m = model_bytes_and_flops(cfg, layers)
    if dtype == torch.float32:  # the true 32-bit path: twice the bytes, CUDA-core kernels
        m["weight_bytes"] *= 2
        m["kv_bytes_per_token"] *= 2
    gen = torch.Generator().manual_seed(1)

    def rand_tokens(n):
        return torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()

    def decode(batch: int, steps: int, warmup: int, sample_clocks: bool = False, context: int = CONTEXT) -> dict:
        """Device time of exactly `steps` decode steps at `batch`, contexts ending at `context`."""
        start_ctx = context - (steps + warmup)
        seqs = list(range(1000, 1000 + batch))
        for s in seqs:
            runner.cache.admit(s, start_ctx)
            runner.cache.commit(s, start_ctx)
        toks = [rand_tokens(steps + warmup) for _ in seqs]
        out = torch.empty(batch, dtype=torch.int32, device="cuda:0")

        def one(i):
            rows = []
            for s, t in zip(seqs, toks):
                runner.cache.extend(s, start_ctx + i + 1)
                rows.append(StepRow(s, [t[i]], start_ctx + i, [0]))
            K.argmax(runner.step(rows), out)

        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        launches0 = K.launch_count()
        clocks = ClockSampler() if sample_clocks else None
        if clocks:
            clocks.__enter__()
            time.sleep(0.3)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        ev0.record()
        for i in range(warmup, warmup + steps):
            one(i)
        ev1.record()
        torch.cuda.synchronize()
        if clocks:
            time.sleep(0.2)
            clocks.__exit__()
        ms = ev0.elapsed_time(ev1) / steps
        for s in seqs:
            runner.cache.release(s)
        mean_ctx = start_ctx + warmup + (steps + 1) / 2  # (of the timed steps)
        nbytes = m["weight_bytes"] + batch * mean_ctx * m["kv_bytes_per_token"]
        return {"ms": ms, "tok_s": batch * 1e3 / ms, "bytes": nbytes, "gbs": nbytes / ms / 1e6,
                "launches": K.launch_count() - launches0,
                "clocks": clocks.summary() if clocks else None}

    def prefill(iters: int = 3, portions: int = 1, ptoks: int = ptoks) -> dict:
        """One prompt of `ptoks` tokens, in one step or in `portions` equal steps."""
        times = []
        part = ptoks // portions
        for it in range(iters + 1):
            runner.cache.admit(5000 + it, ptoks)
            toks = rand_tokens(ptoks)
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            ev0.record()
            for j in range(portions):
                last = j == portions - 1
                runner.step([StepRow(5000 + it, toks[j * part:(j + 1) * part], j * part, [part - 1] if last else [])])
            ev1.record()
            torch.cuda.synchronize()
            runner.cache.release(5000 + it)
            if it:
                times.append(ev0.elapsed_time(ev1))
        ms = statistics.mean(times)
        flops = (ptoks * m["linear_flops_per_token"] + m["attn_flops_causal"](ptoks)
                 + m["head_flops"])
        return {"value": ptoks * 1e3 / ms, "tokens": ptoks, "ms": ms,
                "frac": flops / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), "tflops": flops / ms / 1e9}

    def mixed_step(decoding: int = 32, portion: int = 512, iters: int = 5) -> dict:
        """One step of `decoding` rows that bring one token each (contexts of CONTEXT tokens)
        beside the first `portion` tokens of a new prompt."""
        seqs = list(range(7000, 7000 + decoding))
        for s in seqs:
            runner.cache.admit(s, CONTEXT - iters - 2)
            runner.cache.commit(s, CONTEXT - iters - 2)
        times = []
        for it in range(iters + 1):
            rows = []
            for s in seqs:
                at = CONTEXT - iters - 2 + it
                runner.cache.extend(s, at + 1)
                rows.append(StepRow(s, rand_tokens(1), at, [0]))
            runner.cache.admit(7900 + it, portion)
            rows.append(StepRow(7900 + it, rand_tokens(portion), 0, [portion - 1]))
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            ev0.record()
            runner.step(rows)
            ev1.record()
            torch.cuda.synchronize()
            runner.cache.release(7900 + it)
            if it:
                times.append(ev0.elapsed_time(ev1))
        for s in seqs:
            runner.cache.release(s)
        ms = statistics.mean(times)
        return {"ms": ms, "tok_s": (decoding + portion) * 1e3 / ms}

    def end_to_end(batch: int, steps: int, warmup: int) -> dict:
        """The same decode steps through LLMEngine.step(): schedule, pack, copy in, run,
        sample, copy out, stop-check."""
        ecfg = EngineConfig(dtype=torch.bfloat16, block_size=PAGE_SIZE, max_model_len=CONTEXT + 64,
                            max_num_batched_tokens=8192, max_num_seqs=max_b,
                            enable_cuda_graphs=False)  # the runner's graphs are on already
        engine = LLMEngine.from_runner(runner, ecfg)
        prompt_len = CONTEXT - (steps + warmup) - 1
        for b in range(batch):
            engine.add_request(f"bench-{b}", rand_tokens(prompt_len),
                               SamplingParams(max_tokens=steps + warmup + 8, temperature=0.0, ignore_eos=True))
        while any(r.num_output_tokens == 0 for r in engine.scheduler.running) or engine.scheduler.waiting:
            engine.step()
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        clocks = ClockSampler()
        clocks.__enter__()
        time.sleep(0.3)
        t0 = time.perf_counter()
        produced = 0
        marks = []
        for _ in range(steps):
            produced += len(engine.step())
            marks.append(time.perf_counter())
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        time.sleep(0.2)
        clocks.__exit__()
        if os.environ.get("EMBERSERVE_BENCH_TRACE"):
            print("e2e step ms:", [round((b - a) * 1e3, 2) for a, b in zip([t0] + marks, marks)],
                  "tail", round((t0 + dt - marks[-1]) * 1e3, 2), file=sys.stderr)
        h2d = runner.last_meta_bytes
        engine.reset()
        return {"value": produced / dt, "unit": "tok/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4 * batch, "ms_per_step": dt * 1e3 / steps, "clocks": clocks.summary()}

    def kernel_times(fn) -> list:
        """Device time per kernel name over one call of `fn` (torch's profiler)."""
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            fn()
            torch.cuda.synchronize()
        rows = sorted(prof.key_averages(), key=lambda e: -e.device_time_total)
        total = sum(e.device_time_total for e in rows) or 1.0
        return [{"kernel": e.key[:90], "calls": e.count, "us": round(e.device_time_total, 1),
                 "share": round(e.device_time_total / total, 4)} for e in rows[:25]]

    if args.only == "decode":
        d = decode(args.batch, args.steps, args.warmup, context=args.decode_context)
        out = {"only": "decode", "dtype": args.dtype, "batch": args.batch, "layers": layers,
               "shape": args.model_shape, "context": args.decode_context, "ms_per_step": d["ms"],
               "tok_s": d["tok_s"], "hbm_frac": d["gbs"] / peaks["hbm_gbs"],
               "tiled_weight_copy_gb": round(runner.tiled_weight_bytes / 1e9, 2)}
        if args.kernel_times:
            out["kernels"] = kernel_times(lambda: decode(args.batch, args.steps, args.warmup,
                                                         context=args.decode_context))
        return out
    if args.only == "prefill":
        out = dict(prefill(max(1, args.steps)), only="prefill", layers=layers, dtype=args.dtype)
        if args.kernel_times:
            out["kernels"] = kernel_times(lambda: prefill(1))
        return out
    used_graphs = bool(runner.use_graphs)
    tiled_gb = round(runner.tiled_weight_bytes / 1e9, 2)
    main = decode(args.batch, args.steps, args.warmup, sample_clocks=True)
    pre = prefill()
    b1 = decode(1, min(args.steps, 32), 3)
    b64 = decode(64, min(args.steps, 32), 3)
    half = decode(args.batch, min(args.steps, 32), 3, context=CONTEXT // 2)
    pre4 = prefill(2, portions=4)
    e2e = end_to_end(args.batch, args.steps, args.warmup)
    points = {"decode_b1": b1["tok_s"], "decode_b64": b64["tok_s"],
              f"decode_b{args.batch}_ctx{CONTEXT // 2}": half["tok_s"], "prefill_4x512": pre4["value"],
              "decode_b1_hbm_frac": b1["gbs"] / peaks["hbm_gbs"],
              "decode_b64_hbm_frac": b64["gbs"] / peaks["hbm_gbs"]}
    for t in (128, 256, 512):
        short = prefill(3, ptoks=t)
        points[f"prefill_{t}"] = short["value"]
        # a short prompt step is bound by the weights it reads, not by arithmetic
        points[f"prefill_{t}_hbm_frac"] = m["weight_bytes"] / short["ms"] / 1e6 / peaks["hbm_gbs"]
    mixed = mixed_step()
    points["mixed_32dec_512prefill_tok_s"] = mixed["tok_s"]
    points["mixed_32dec_512prefill_ms"] = mixed["ms"]
    # the reference's own profiled mixed step (docs/results.md:452-459: 39 decode rows beside a
    # 300-token chunk, 27.25 ms of GPU time on an A100 in fp16), here with contexts of 4096
    points["mixed_39dec_300prefill_ms"] = mixed_step(39, 300)["ms"]
    if not args.no_extras:
        # free this model before others are built (the child processes need the memory)
        runner.graphs = None
        del runner
        import gc

        gc.collect()
        torch.cuda.empty_cache()
        points.update(kernel_points(args))
        points.update(extra_points(args))
    return {
        "metric": "decode tok/s at batch 8, context 4096 (Qwen2.5-7B shape)",
        "value": main["tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": main["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform random token ids, random weights N(0,0.02) seed 0",
        "impl": "ours",
        "config": {"model": "Qwen2.5-7B shape", "layers": layers, "layers_full": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": args.batch, "seq_len": CONTEXT, "page_size": PAGE_SIZE,
                   "prefill_tokens": PREFILL_TOKENS, "parallelism": "1gpu",
                   "l2": "inputs larger than L2", "cuda_graphs": used_graphs,
                   "tiled_weight_copy_gb": tiled_gb, "peaks": peaks["source"]},
        "clocks": main["clocks"], "gpu_launches": main["launches"], "e2e": e2e,
        "prefill": pre,
        "roofline": {"bound": "hbm", "achieved": main["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": main["gbs"] / peaks["hbm_gbs"]},
        "points": points,
        "reference_a100_fp16_b8_tok_s": A100_FP16_B8_TOK_S,
    }


def kernel_points(args) -> dict:
    """The kernels that a step's time goes to, each alone at the 7B geometry (`run_kernel`), as
    fractions of the measured peaks: the four projections at 8 rows, the decode attention at
    batch 8 and 64, the prompt attention of 2,048 tokens."""
    import copy

    out = {}

    def one(**kw):
        a = copy.copy(args)
        a.model_shape, a.splits, a.start, a.attn_kernel, a.steps = "7b", 0, 0, "auto", 5
        for key, value in kw.items():
            setattr(a, key, value)
        return run_kernel(a)

    for shape in ("qkv", "o", "gate_up", "down"):
        r = one(kernel="gemm", shape=shape, batch=8)
        out[f"kernel_{shape}_m8_hbm_frac"] = r["frac_hbm"]
        out[f"kernel_{shape}_m8_us"] = r["ms"] * 1e3
    for b in (8, 64):
        r = one(kernel="decode_attention", batch=b, context=CONTEXT, fused=True)
        out[f"kernel_decode_attention_b{b}_hbm_frac"] = r["frac_hbm"]
        out[f"kernel_decode_attention_b{b}_us"] = r["ms"] * 1e3
    r = one(kernel="prefill_attention", context=PREFILL_TOKENS)
    out["kernel_prefill_attention_2048_bf16_frac"] = r["frac_bf16"]
    out["kernel_prefill_attention_2048_us"] = r["ms"] * 1e3
    return out


def extra_points(args) -> dict:
    """The measurements that need another model: each in a child process of this script (its own
    CUDA context, freed when it exits), one after the other.  A child that fails leaves a note
    instead of its numbers; the headline does not depend on them."""
    out = {}

    def child(*flags, timeout=600):
        cmd = [sys.executable, str(ROOT / "bench.py"), "--steps", "32", "--warmup", "3", *flags]
        try:
            proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
            lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
            if proc.returncode != 0 or not lines:
                return {"error": (proc.stderr or proc.stdout)[-200:].replace("\n", " ")}
            return json.loads(lines[-1])
        except Exception as e:  # a time-out, or output that is no JSON
            return {"error": f"{type(e).__name__}: {e}"[:200]}

    r = child("--workload", "fp32-7b")
    if "error" in r:
        out["fp32_error"] = r["error"]
    else:
        out.update({k: v for k, v in r.items() if k.startswith("fp32_")})
    # (wall-clock through LLM.generate: the host's share of a 2 ms step is large, and so is the
    # spread between runs on a shared host; two runs, the better one and the other)
    runs = [child("--workload", "serve-0.5b") for _ in range(2)]
    good = sorted((r for r in runs if "value" in r), key=lambda r: -r["value"])
    if good:
        out["serve_0.5b_tok_s"] = good[0]["value"]
        out["serve_0.5b_requests"] = good[0]["requests"]
        if len(good) > 1:
            out["serve_0.5b_tok_s_other_run"] = good[1]["value"]
    else:
        out["serve_0.5b_error"] = runs[0].get("error")
    r = child("--workload", "mixed-32b", timeout=900)
    out["mixed_32b_tok_s" if "value" in r else "mixed_32b_error"] = r.get("value", r.get("error"))
    if "value" in r:
        out["mixed_32b_ms_per_step"] = r["ms_per_step_wall"]
    return out


def run_fp32(args) -> dict:
    """The true 32-bit path at the 7B shape (float32 weights, cache and activations, SGEMM with
    TF32 off, CUDA-core attention): decode at batch 1 and 8, and the 2,048-token prefill, with
    the fractions of the measured copy bandwidth (the prefill as a rate: the denominator that
    would apply, SGEMM's own peak, is not measured here)."""
    import copy

    a = copy.copy(args)
    a.dtype, a.model_shape, a.only, a.kernel_times, a.layers = "float32", "7b", "decode", False, None
    import gc

    import torch

    out = {}
    for b in (1, 8):
        a.batch, a.decode_context = b, CONTEXT
        r = run_ours(a)
        out[f"fp32_decode_b{b}"] = r["tok_s"]
        out[f"fp32_decode_b{b}_hbm_frac"] = r["hbm_frac"]
        gc.collect()  # (the 30 GB of the model that has just been timed)
        torch.cuda.empty_cache()
    a.only, a.prefill_tokens, a.steps = "prefill", PREFILL_TOKENS, 2
    r = run_ours(a)
    out["fp32_prefill_2048"] = r["value"]
    out["fp32_prefill_2048_tflops"] = r["tflops"]
    out["fp32_prefill_2048_frac_of_bf16_peak"] = r["frac"]
    return out


def run_kernel(args) -> dict:
    """One kernel alone at the geometry of the 7B shape, inputs larger than L2, timed with
    CUDA events (median of the iterations): achieved bandwidth or arithmetic rate against
    the measured peaks.  This is also the small case that ncu profiles are taken on."""
    import math

    import torch

    from emberserve_b200 import kernels as K

    peaks = measured_peaks()
    s = {"7b": SHAPE_7B, "0.5b": SHAPE_05B, "32b": SHAPE_32B}[args.model_shape]
    nh, nkv, d, ps = s["num_attention_heads"], s["num_key_value_heads"], s["head_dim"], PAGE_SIZE
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(0)
    iters = max(3, args.steps)

    def timed(fn, reps: int = 8) -> float:
        """Median device time of one call.  `reps` calls are captured in a CUDA graph and the
        replay is timed, so that the host's launch cost is not what is measured; every call
        of a replay reads its inputs again from memory (they exceed L2 where it matters)."""
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                fn()
        graph.replay()
        times = []
        for _ in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) / reps)
        return statistics.median(times)

    if args.kernel == "decode_attention":
        # the attention of one layer of a decode step: rotation of q and k, write of the new key
        # and value, attention over the cache (and the merge of the key splits), either as the
        # three kernels of the unfused path or as the one fused kernel (--fused)
        b, ctx = args.batch, args.context
        width = ctx // ps + 1
        pages = b * width
        nbytes = 2 * b * ctx * nkv * d * 2
        copies = max(2, int(300e6 // nbytes) + 1)  # used in turn, so that no key is found in L2
        caches = [(torch.randn(pages, nkv, ps, d, device=dev, generator=g).to(torch.bfloat16),
                   torch.randn(pages, nkv, ps, d, device=dev, generator=g).to(torch.bfloat16)) for _ in range(copies)]
        bt = torch.randperm(pages, device=dev, generator=g).view(b, width).to(torch.int32)
        qkv = torch.randn(b, (nh + 2 * nkv) * d, device=dev, generator=g).to(torch.bfloat16)
        out = torch.empty(b, nh * d, device=dev, dtype=torch.bfloat16)
        cu = torch.arange(b + 1, device=dev, dtype=torch.int32)
        st = torch.full((b,), ctx - 1, device=dev, dtype=torch.int32)
        if args.varied_context:  # requests of a serving batch: contexts spread evenly over 64..ctx
            st = torch.randint(63, ctx, (b,), device=dev, generator=g).to(torch.int32)
            nbytes = 2 * int((st.long() + 1).sum()) * nkv * d * 2
        rows = torch.arange(b, device=dev, dtype=torch.int32)
        from emberserve_b200.parts.attention import decode_splits
        from emberserve_b200.parts.rope import inv_frequencies

        table = K.rope_table(inv_frequencies(d, 1e6).to(dev), ctx + 1)
        splits = args.splits or decode_splits(b, nkv, ctx)
        scratch = torch.empty(max(1, K.attention_scratch_bytes(b, nh, d, splits) // 4), device=dev)
        state = {"i": 0}

        def unfused():
            kc, vc = caches[state["i"] % copies]
            state["i"] += 1
            K.rope_kv_write(qkv, nh, nkv, d, st, rows, table, d, kc, vc, bt, ps)
            K.paged_attention(qkv, out, kc, vc, bt, cu, st, b, b, nh, nkv, d, 1 / math.sqrt(d), 1, splits=splits,
                              scratch=scratch)

        def fused():
            kc, vc = caches[state["i"] % copies]
            state["i"] += 1
            K.decode_attention_fused(qkv, out, kc, vc, bt, cu, st, b, nh, nkv, d, 1 / math.sqrt(d), table, d, True,
                                     splits=splits, scratch=scratch)

        ms = timed(fused if args.fused else unfused, reps=copies)
        return {"kernel": "decode_attention", "fused": bool(args.fused), "batch": b, "context": ctx,
                "splits": splits, "ms": ms, "gbs": nbytes / ms / 1e6,
                "frac_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"], "bytes": nbytes}
    if args.kernel == "prefill_attention":
        t, s0 = args.context, args.start  # a portion of t tokens behind s0 cached keys
        width = (s0 + t) // ps + 1
        kc = torch.randn(width, nkv, ps, d, device=dev, generator=g).to(torch.bfloat16)
        vc = torch.randn(width, nkv, ps, d, device=dev, generator=g).to(torch.bfloat16)
        bt = torch.randperm(width, device=dev, generator=g).view(1, width).to(torch.int32)
        qkv = torch.randn(t, (nh + 2 * nkv) * d, device=dev, generator=g).to(torch.bfloat16)
        out = torch.empty(t, nh * d, device=dev, dtype=torch.bfloat16)
        cu = torch.tensor([0, t], device=dev, dtype=torch.int32)
        st = torch.full((1,), s0, device=dev, dtype=torch.int32)
        ms = timed(lambda: K.paged_attention(qkv, out, kc, vc, bt, cu, st, 1, t, nh, nkv, d,
                                             1 / math.sqrt(d), t, kernel=args.attn_kernel))
        K.check_status()
        flops = 4 * nh * d * (t * s0 + t * t / 2)
        return {"kernel": "prefill_attention", "impl": args.attn_kernel, "tokens": t, "start": s0, "ms": ms,
                "tflops": flops / ms / 1e9, "frac_bf16": flops / ms / 1e9 / peaks["bf16_tflops"]}
    if args.kernel == "gemm":
        h, i, v = s["hidden_size"], s["intermediate_size"], s["vocab_size"]
        shapes = {"qkv": ((nh + 2 * nkv) * d, h), "o": (h, nh * d), "gate_up": (2 * i, h), "down": (h, i),
                  "head": (v, h)}
        n_out, k = shapes[args.shape]
        m = args.batch
        # several copies of the weight, used in turn, so that it is never found in L2
        copies = max(2, int(300e6 // (n_out * k * 2)) + 1)
        ws = [(torch.randn(n_out, k, device=dev, generator=g) * 0.02).to(torch.bfloat16) for _ in range(copies)]
        x = torch.randn(m, k, device=dev, generator=g).to(torch.bfloat16)
        out = torch.empty(m, n_out, device=dev, dtype=torch.bfloat16)
        if m > 64 and (args.shape == "gate_up" or m > 128):
            # prompt portions: the two-SM gated kernel against cuBLAS and its activation kernel
            if args.shape != "gate_up":
                raise SystemExit("with more than 128 rows only --shape gate_up has a kernel of its own "
                                 "(the plain products of prompt steps are the library's)")
            act = torch.empty(m, n_out // 2, device=dev, dtype=torch.bfloat16)
            st = {"i": 0}

            twins = [K.tile_weight(w) for w in ws]

            def ours_large():
                K.gemm_large_gated(x, ws[st["i"] % copies], act)
                st["i"] += 1

            def ours_large_tiled():
                K.gemm_large_gated(x, ws[st["i"] % copies], act, twin=twins[st["i"] % copies])
                st["i"] += 1

            def lib_large():
                torch.mm(x, ws[st["i"] % copies].t(), out=out)
                if args.shape == "gate_up":
                    K.silu_mul(out, act)
                st["i"] += 1

            ms = timed(ours_large, reps=copies)
            ms_tiled = timed(ours_large_tiled, reps=copies)
            ms_lib = timed(lib_large, reps=copies)
            K.check_status()
            flops = 2.0 * m * n_out * k
            return {"kernel": "gemm", "shape": args.shape, "m": m, "n": n_out, "k": k, "ms": ms,
                    "tflops": flops / ms / 1e9, "frac_bf16": flops / ms / 1e9 / peaks["bf16_tflops"],
                    "ms_tiled_copy": ms_tiled, "cublas_ms": ms_lib, "cublas_tflops": flops / ms_lib / 1e9}
        from emberserve_b200.parts.linear import midm_ksplit, smallm_ksplit

        if m > 16 and args.shape != "gate_up":  # the kernel for 17..128 rows
            ksplit = args.splits or midm_ksplit(m, n_out, k)
            st = {"i": 0}

            twins = [K.tile_weight(w) for w in ws]  # as the engine runs it: from the tiled copy

            def mid():
                K.gemm_midm(x, ws[st["i"] % copies], None, out, ksplit=ksplit, twin=twins[st["i"] % copies])
                st["i"] += 1

            def lib():
                torch.mm(x, ws[st["i"] % copies].t(), out=out)
                st["i"] += 1

            ms, ms_lib = timed(mid, reps=copies), timed(lib, reps=copies)
            K.check_status()
            nbytes = n_out * k * 2
            return {"kernel": "gemm", "shape": args.shape, "m": m, "n": n_out, "k": k, "ksplit": ksplit, "ms": ms,
                    "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"],
                    "cublas_ms": ms_lib, "cublas_gbs": nbytes / ms_lib / 1e6}
        ksplit = args.splits or smallm_ksplit(m, n_out, k)
        act = torch.empty(m, n_out // 2, device=dev, dtype=torch.bfloat16)
        state = {"i": 0}

        twins = [None if args.no_tiled_weights else K.tile_weight(w) for w in ws]

        def ours():
            i = state["i"] % copies
            if args.shape == "gate_up":  # as the engine runs it: both halves and SiLU in one kernel
                K.gemm_smallm_gated(x, ws[i], act, twin=twins[i])
            else:
                K.gemm_smallm(x, ws[i], None, out, ksplit=ksplit, twin=twins[i])
            state["i"] += 1

        def cublas():
            torch.mm(x, ws[state["i"] % copies].t(), out=out)
            state["i"] += 1

        ms = timed(ours, reps=copies)
        ms_lib = timed(cublas, reps=copies)
        K.check_status()
        nbytes = n_out * k * 2
        return {"kernel": "gemm", "shape": args.shape, "m": m, "n": n_out, "k": k, "ksplit": ksplit, "ms": ms,
                "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"],
                "cublas_ms": ms_lib, "cublas_gbs": nbytes / ms_lib / 1e6}
    raise SystemExit(f"unknown kernel {args.kernel!r}")


SHAPE_05B = dict(vocab_size=151936, hidden_size=896, intermediate_size=4864, num_hidden_layers=24,
                 num_attention_heads=14, num_key_value_heads=2, head_dim=64, max_position_embeddings=32768,
                 rms_norm_eps=1e-6, rope_theta=1_000_000.0, tie_word_embeddings=True, attention_bias=True,
                 eos_token_id=151645)


def run_serving(args) -> dict:
    """Continuous batching of many requests through LLM.generate(): 256 requests with
    uniform-random prompts of 64..1024 tokens and 128..512 output tokens each, Qwen2.5-0.5B
    shape, bfloat16, random weights.  Wall clock around the whole generate() call, the second of two
    identical calls in the process (`first_pass_seconds` is the first)."""
    import random

    import torch

    from emberserve_b200 import kernels as K
    from emberserve_b200.config.engine import EngineConfig
    from emberserve_b200.config.model import Qwen2Config
    from emberserve_b200.engine.llm_engine import LLMEngine
    from emberserve_b200.engine.runner import ModelRunner
    from emberserve_b200.llm import LLM
    from emberserve_b200.sampling.params import SamplingParams

    cfg = Qwen2Config.from_dict(dict(SHAPE_05B, architectures=["Qwen2ForCausalLM"], model_type="qwen2"))
    K.library()
    n_req = args.requests
    rng = random.Random(0)
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(rng.randint(64, 1024))] for _ in range(n_req)]
    params = [SamplingParams(max_tokens=rng.randint(128, 512), temperature=args.temperature, top_k=args.top_k,
                             top_p=args.top_p, seed=i, ignore_eos=True) for i in range(n_req)]
    max_len = 2048
    pages = n_req * (max_len // PAGE_SIZE) + 64
    runner = ModelRunner.from_random(cfg, seed=0, dtype=torch.bfloat16, device="cuda:0", page_size=PAGE_SIZE,
                                     num_pages=pages)
    ecfg = EngineConfig(dtype=torch.bfloat16, block_size=PAGE_SIZE, max_model_len=max_len, max_num_seqs=256,
                        max_num_batched_tokens=2048, enable_chunked_prefill=True,
                        async_scheduling=not args.sync_steps)
    engine = LLMEngine.from_runner(runner, ecfg)
    engine.keep_stats = True
    llm = LLM.from_engine(engine)
    # Warm-up: the whole workload once.  Its steps have every row count between 1 and 256, and the
    # first product of each row count makes the library load (and choose) a kernel for it, which
    # costs tens of milliseconds each: a server pays that once, in its first seconds.
    t0 = time.perf_counter()
    llm.generate(prompts, params)
    torch.cuda.synchronize()
    first = time.perf_counter() - t0
    engine.stats.clear()
    with ClockSampler() as clocks:
        t0 = time.perf_counter()
        results = llm.generate(prompts, params)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    out_tokens = sum(len(r.output_token_ids) for r in results)
    in_tokens = sum(len(p) for p in prompts)
    fwd = sorted(s.forward_ms + s.sample_ms for s in engine.stats)
    return {"metric": "output tok/s, continuous batching of 256 requests (Qwen2.5-0.5B shape)",
            "value": out_tokens / dt, "unit": "tok/s", "n_gpus": 1, "seconds": dt,
            "first_pass_seconds": first, "requests": n_req,
            "output_tokens": out_tokens, "prompt_tokens": in_tokens, "steps": len(engine.stats),
            "step_ms_p50": fwd[len(fwd) // 2], "step_ms_p99": fwd[int(len(fwd) * 0.99)],
            "ms_per_step_wall": dt * 1e3 / max(1, len(engine.stats)),
            "host_launch_seconds": sum(fwd) / 1e3,
            "preemptions": sum(s.num_preempted for s in engine.stats), "dtype": "bf16",
            "data": "synthetic: uniform random token ids and lengths (seed 0), random weights",
            "sampling": {"temperature": args.temperature, "top_k": args.top_k, "top_p": args.top_p},
            "config": {"model": "Qwen2.5-0.5B shape", "layers": cfg.num_hidden_layers, "max_num_seqs": 256,
                       "max_num_batched_tokens": 2048, "page_size": PAGE_SIZE}, "clocks": clocks.summary()}


SHAPE_32B = dict(vocab_size=152064, hidden_size=5120, intermediate_size=27648, num_hidden_layers=64,
                 num_attention_heads=40, num_key_value_heads=8, head_dim=128, max_position_embeddings=32768,
                 rms_norm_eps=1e-5, rope_theta=1_000_000.0, tie_word_embeddings=False, attention_bias=True)


def run_mixed_32b(args) -> dict:
    """Chunked prefill of long prompts beside decoding requests at the Qwen2.5-32B shape: 32
    requests with prompts of 8192 uniform-random tokens and 32 output tokens each, a token budget
    of 2048 per step, through LLM.generate(); bfloat16, random weights (65.5 GB) and 69 GB of keys
    and values.  Wall clock around the whole call; the steps that only decode are timed apart."""
    import random

    import torch

    from emberserve_b200 import kernels as K
    from emberserve_b200.config.engine import EngineConfig
    from emberserve_b200.config.model import Qwen2Config
    from emberserve_b200.engine.llm_engine import LLMEngine
    from emberserve_b200.engine.runner import ModelRunner
    from emberserve_b200.llm import LLM
    from emberserve_b200.sampling.params import SamplingParams

    cfg = Qwen2Config.from_dict(dict(SHAPE_32B, architectures=["Qwen2ForCausalLM"], model_type="qwen2"))
    K.library()
    n_req, prompt_len, out_len = args.requests if args.requests != 256 else 32, 8192, 32
    rng = random.Random(0)
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(prompt_len)] for _ in range(n_req)]
    params = SamplingParams(max_tokens=out_len, temperature=0.0, ignore_eos=True)
    max_len = prompt_len + out_len + 16
    pages = n_req * (max_len // PAGE_SIZE + 1) + 64
    runner = ModelRunner.from_random(cfg, seed=0, dtype=torch.bfloat16, device="cuda:0", page_size=PAGE_SIZE,
                                     num_pages=pages)
    ecfg = EngineConfig(dtype=torch.bfloat16, block_size=PAGE_SIZE, max_model_len=max_len, max_num_seqs=n_req,
                        max_num_batched_tokens=2048, enable_chunked_prefill=True)
    engine = LLMEngine.from_runner(runner, ecfg)
    engine.keep_stats = True
    llm = LLM.from_engine(engine)
    llm.generate([prompts[0][:300]], [SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True)])  # warm-up
    engine.stats.clear()
    torch.cuda.synchronize()
    with ClockSampler() as clocks:
        t0 = time.perf_counter()
        results = llm.generate(prompts, params)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    out_tokens = sum(len(r.output_token_ids) for r in results)
    mixed = [s for s in engine.stats if s.num_prefill_tokens and s.num_decode_tokens]
    return {"metric": "chunked prefill beside decode, 32 requests of 8192 prompt tokens (Qwen2.5-32B shape)",
            "value": (n_req * prompt_len + out_tokens) / dt, "unit": "tok/s (prompt + output)", "n_gpus": 1,
            "seconds": dt, "requests": n_req, "prompt_tokens": n_req * prompt_len, "output_tokens": out_tokens,
            "steps": len(engine.stats), "mixed_steps": len(mixed),
            "ms_per_step_wall": dt * 1e3 / max(1, len(engine.stats)), "dtype": "bf16",
            "data": "synthetic: uniform random token ids (seed 0), random weights",
            "config": {"model": "Qwen2.5-32B shape", "layers": cfg.num_hidden_layers, "max_num_seqs": n_req,
                       "max_num_batched_tokens": 2048, "page_size": PAGE_SIZE, "prompt_len": prompt_len,
                       "output_len": out_len}, "clocks": clocks.summary()}


def run_reference(args) -> dict:
    """The unmodified reference, installed under baseline/_ref, through its own LLMEngine."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "emberserve").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref holds no install of the reference"}
    sys.path.insert(0, str(ref))
    try:
        import torch
        from emberserve.config import EngineConfig, ModelConfig
        from emberserve.engine import LLMEngine
        from emberserve.model.qwen2 import Qwen2ForCausalLM
        from emberserve.sched.request import SamplingParams
    except Exception as e:  # pragma: no cover - depends on the machine
        return {"impl": "reference", "unavailable": f"import failed: {type(e).__name__}: {e}"[:300]}
    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA GPU"}
    s = SHAPE_7B
    mcfg = ModelConfig(
        vocab_size=s["vocab_size"], hidden_size=s["hidden_size"], intermediate_size=s["intermediate_size"],
        num_hidden_layers=args.layers or s["num_hidden_layers"], num_attention_heads=s["num_attention_heads"],
        num_key_value_heads=s["num_key_value_heads"], max_position_embeddings=s["max_position_embeddings"],
        rms_norm_eps=s["rms_norm_eps"], rope_theta=s["rope_theta"],
        tie_word_embeddings=s["tie_word_embeddings"], attention_bias=s["attention_bias"],
        eos_token_id=s["eos_token_id"])
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device("cuda"):
            model = Qwen2ForCausalLM(mcfg, tp_size=1)
    finally:
        torch.set_default_dtype(prev)
    with torch.no_grad():
        gen = torch.Generator(device="cuda").manual_seed(0)
        for name, p in model.named_parameters():
            if "norm" in name:
                p.fill_(1.0)
            else:
                p.normal_(0, 0.02, generator=gen)
    errors = []
    for backend, block, graphs in (("paged_triton", 16, True), ("paged_triton", 16, False),
                                   ("paged_flash", 256, True), ("paged_flash", 256, False),
                                   ("paged_torch", 16, False)):
        try:
            pages = 80 * (CONTEXT // block + 2)
            ecfg = EngineConfig(device="cuda", dtype=torch.bfloat16, attn_backend=backend, block_size=block,
                                num_gpu_blocks=pages, max_num_seqs=64, max_num_batched_tokens=8192,
                                max_model_len=CONTEXT + 64, enable_cuda_graphs=graphs,
                                enable_chunked_prefill=True)
            engine = LLMEngine(model, mcfg, ecfg, tokenizer=None)
            engine.keep_stats = False
            g = torch.Generator().manual_seed(1)
            prompt_len = CONTEXT - (args.steps + args.warmup) - 1
            for b in range(args.batch):
                ids = torch.randint(0, mcfg.vocab_size, (prompt_len,), generator=g).tolist()
                engine.add_request(f"bench-{b}", ids, SamplingParams(
                    max_tokens=args.steps + args.warmup + 8, temperature=0.0, ignore_eos=True))
            while engine.scheduler.waiting or any(r.num_output_tokens == 0 for r in engine.scheduler.running):
                engine.step()
            for _ in range(args.warmup):
                engine.step()
            torch.cuda.synchronize()
            with ClockSampler() as clocks:
                t0 = time.perf_counter()
                produced = 0
                for _ in range(args.steps):
                    produced += len(engine.step())
                torch.cuda.synchronize()
                dt = time.perf_counter() - t0
            return {"metric": "decode tok/s at batch 8, context 4096 (Qwen2.5-7B shape)",
                    "value": produced / dt, "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
                    "warmup": args.warmup, "ms_per_step": dt * 1e3 / args.steps, "higher_is_better": True,
                    "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                    "impl": "reference",
                    "config": {"model": "Qwen2.5-7B shape", "layers": mcfg.num_hidden_layers,
                               "global_batch": args.batch, "seq_len": CONTEXT, "attn_backend": backend,
                               "block_size": block, "cuda_graphs": graphs, "parallelism": "1gpu"},
                    "clocks": clocks.summary(),
                    "e2e": {"value": produced / dt, "unit": "tok/s"},
                    "tried": errors}
        except Exception as e:  # try the next stock backend of the reference
            errors.append(f"{backend}/graphs={graphs}: {type(e).__name__}: {str(e)[:120]}")
            torch.cuda.synchronize()
    return {"impl": "reference", "unavailable": "no attention backend of the reference ran here: "
            + " | ".join(errors)[:600]}


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--workload", choices=["decode-7b", "serve-0.5b", "mixed-32b", "fp32-7b"], default="decode-7b",
                    help="decode-7b: the headline line; serve-0.5b: continuous batching of --requests requests; "
                         "mixed-32b: chunked prefill of long prompts beside decode at the 32B shape; fp32-7b: "
                         "the true 32-bit path (the headline line runs the last three as child processes)")
    ap.add_argument("--no-extras", action="store_true",
                    help="the headline line without the points that need other models or kernels alone")
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--varied-context", action="store_true",
                    help="with --kernel decode_attention: contexts spread evenly over 64..--context")
    ap.add_argument("--no-graphs", action="store_true", help="run decode steps eagerly")
    ap.add_argument("--no-tiled-weights", action="store_true",
                    help="without the engine's second, tiled copy of the projection weights (by default it is "
                         "made where it takes at most a tenth of the device's memory, as here)")
    ap.add_argument("--only", choices=["decode", "prefill", "kernel"], default=None,
                    help="run one small part only (for profiling): decode at --batch, the prefill, or "
                         "one kernel alone (--kernel)")
    ap.add_argument("--kernel", choices=["decode_attention", "prefill_attention", "gemm"],
                    default="decode_attention")
    ap.add_argument("--shape", choices=["qkv", "o", "gate_up", "down", "head"], default="qkv",
                    help="with --kernel gemm: which projection of the 7B shape")
    ap.add_argument("--context", type=int, default=CONTEXT, help="with --only kernel: keys (or prompt tokens)")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                    help="with --only decode / prefill: float32 times the true 32-bit path (the line's "
                         "prefill fraction stays relative to the bfloat16 peak)")
    ap.add_argument("--sync-steps", action="store_true",
                    help="with --workload serve-0.5b: read every step's tokens before the next is planned")
    ap.add_argument("--temperature", type=float, default=0.0, help="with --workload serve-0.5b (0 = greedy)")
    ap.add_argument("--top-k", type=int, default=-1, help="with --workload serve-0.5b")
    ap.add_argument("--top-p", type=float, default=1.0, help="with --workload serve-0.5b")
    ap.add_argument("--model-shape", choices=["7b", "0.5b", "32b"], default="7b",
                    help="with --only decode / prefill: the layer sizes (the default line is always the 7B shape)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="with --only prefill: the prompt's length")
    ap.add_argument("--decode-context", type=int, default=CONTEXT, help="with --only decode: context the steps end at")
    ap.add_argument("--library-prefill-mlp", action="store_true",
                    help="for comparison: gate/up product of prompt steps by cuBLAS and a separate SiLU "
                         "kernel instead of the two-SM tcgen05 kernel with SiLU in its epilogue")
    ap.add_argument("--fused", action="store_true",
                    help="with --kernel decode_attention: the fused kernel instead of the three")
    ap.add_argument("--start", type=int, default=0,
                    help="with --kernel prefill_attention: keys cached before the portion")
    ap.add_argument("--splits", type=int, default=0, help="with --only kernel: key splits (0 = the engine's rule)")
    ap.add_argument("--attn-kernel", choices=["auto", "mma", "tcgen05", "generic"], default="auto",
                    help="with --kernel prefill_attention: which of the attention kernels")
    ap.add_argument("--kernel-times", action="store_true",
                    help="with --only: add device time per kernel name (torch profiler)")
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the shape has (the line then names both numbers)")
    args = ap.parse_args()
    if args.library_prefill_mlp:
        from emberserve_b200 import kernels as _K

        _K.gemm_large_gated_supported = lambda m, inter, k: False
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py measures a one-GPU engine; --gpus {args.gpus} is not supported (N=1 only)")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.only == "kernel":
        print(json.dumps(run_kernel(args)))
        return 0
    if args.workload == "serve-0.5b":
        print(json.dumps(run_serving(args)))
        return 0
    if args.workload == "mixed-32b":
        print(json.dumps(run_mixed_32b(args)))
        return 0
    if args.workload == "fp32-7b":
        print(json.dumps(run_fp32(args)))
        return 0
    result = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
