#!/usr/bin/env python3
"""Headline benchmark: decode tokens/s of the Llama-3.2-1B shape in bfloat16 on one
B200 (batch 8 at the stated context length), with prefill of 2,048 tokens, decode
at batch 1 and 64, the same metric end to end through the Python entry point, and
roofline fractions.  Prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

A "step" is one decode step of the whole batch (model forward over the paged
cache plus on-device sampling).  Weights are random (seeded normal, std 0.02),
token ids are seeded uniform: there is no network for checkpoints or datasets.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# the headline configuration: the Llama-3.2-1B shape
LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 16, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
    "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "max_position_embeddings": 131072, "tie_word_embeddings": True,
}
# the other shapes that the reference's benchmark configurations name (--shape, for measurements
# beside the headline; the default run is the 1B shape)
LLAMA_3B = dict(LLAMA_1B, num_hidden_layers=28, hidden_size=3072, num_attention_heads=24, head_dim=128)
LLAMA_8B = dict(LLAMA_1B, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, head_dim=128,
                intermediate_size=14336, tie_word_embeddings=False,
                rope_scaling=dict(LLAMA_1B["rope_scaling"], factor=8.0))
SHAPES = {"1b": ("Llama-3.2-1B", LLAMA_1B), "3b": ("Llama-3.2-3B", LLAMA_3B), "8b": ("Llama-3.1-8B", LLAMA_8B)}
CONTEXT = 8192
BATCH = 8
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}

REFERENCE_UNAVAILABLE = ("hvasconcelos/mlxforge builds only on Apple (CMakeLists.txt:14-16 errors elsewhere) and "
                         "computes through Apple MLX/Metal, which this box does not have; it has no pip package")


def peaks():
    """HBM copy bandwidth and the library's bfloat16 product throughput as a burst (the divisor for
    a region of a few milliseconds timed alone between synchronisations, as the prefill here is)
    and sustained under the power cap."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                j = json.load(f)
            hbm, burst = j.get("hbm_gbs"), j.get("bf16_tflops")
            if hbm and burst:
                return {"hbm_gbs": float(hbm), "bf16_tflops": float(burst),
                        "bf16_tflops_sustained": float(j.get("bf16_tflops_sustained") or burst), "source": "measured"}
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi sampling SM clocks and throttle reasons while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None

    def start(self):
        exe = shutil.which("nvidia-smi")
        if not exe:
            return
        self.f = open(self.path, "w")
        self.proc = subprocess.Popen([exe, "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                      "-lms", "100"], stdout=self.f, stderr=subprocess.DEVNULL)

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            with open(self.path) as f:
                for line in f:
                    c = [x.strip() for x in line.split(",")]
                    if len(c) < 7:
                        continue
                    try:
                        sm.append(float(c[0]))
                        mx.append(float(c[1]))
                    except ValueError:
                        continue
                    for n, v in zip(names, c[3:7]):
                        if v.lower().startswith("active"):
                            reasons.add(n)
            os.remove(self.path)
        except OSError:
            pass
        if sm:
            out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons)}
        return out


def decode_device(engine, batch, ctx, steps, warmup, seed=0, segments=5):
    """Device-timed decode: `batch` sequences whose cache holds ~ctx tokens (filled
    with random keys and values, no forward pass needed for that), `warmup` + `steps`
    decode steps of the step function with greedy sampling on the device.  The `steps`
    timed steps are one region between two events; events in between cut it into
    `segments` pieces whose ms per step show the spread.  Returns (seconds per step,
    kernel launches per step, cache tokens read per step, [ms per step of every piece])."""
    import numpy as np
    import torch
    from mlxforge_b200.csrc import binding, ops
    from mlxforge_b200.engine.step import StepEntry
    runner, cache = engine.runner, engine.cache
    rng = np.random.default_rng(seed)
    vocab = engine.model.spec.vocab_size
    start_len = ctx - (warmup + steps)
    seqs = [cache.open_sequence() for _ in range(batch)]
    for s in seqs:
        cache.reserve([(s, start_len)])
        cache.commit(s, start_len)
    out = torch.empty(batch, dtype=torch.int32, device="cuda")
    toks = rng.integers(0, vocab, size=(warmup + steps, batch))

    def one(i):
        logits = runner.step([StepEntry(s, [int(toks[i, b])], [0]) for b, s in enumerate(seqs)])
        ops.sample(logits, None, None, out)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    l0 = binding.launch_count()
    segments = max(1, min(segments, steps))
    cuts = [round(k * steps / segments) for k in range(segments + 1)]
    events = [torch.cuda.Event(enable_timing=True) for _ in cuts]
    events[0].record()
    for k in range(segments):
        for i in range(warmup + cuts[k], warmup + cuts[k + 1]):
            one(i)
        events[k + 1].record()
    torch.cuda.synchronize()
    ops.check_kernel_status()
    sec = events[0].elapsed_time(events[-1]) / 1e3 / steps
    pieces = [events[k].elapsed_time(events[k + 1]) / (cuts[k + 1] - cuts[k]) for k in range(segments)]
    launches = (binding.launch_count() - l0) / steps
    mean_ctx = start_len + warmup + (steps + 1) / 2.0
    for s in seqs:
        cache.close(s)
    return sec, launches, mean_ctx * batch, pieces


def prefill_products_device(engine, tokens, runs=5, warmup=3):
    """The matrix products of a prefill of `tokens` tokens alone (every layer's QKV, output,
    gate|up with its gated epilogue, down; the head's one row is left out), through the same
    dispatch the model uses, on scratch operands.  Returns (seconds, FLOPs)."""
    import torch
    rt = engine.model.rt
    blocks = [engine.model.blocks[item.layer] for item in engine.model.spec.schedule]
    flops = 0.0
    plan = []
    for b in blocks:
        m, f = b.mixer, b.feed_forward
        xs = {}
        for w in (m.w_qkv, m.w_o, f.w_gu, f.w_down):
            k = w.shape[1]
            if k not in xs:
                xs[k] = torch.randn((tokens, k), device=rt.device).to(torch.bfloat16)
            flops += 2.0 * tokens * w.shape[0] * k
        plan.append((m, f, xs))
    outs = {}

    def out(name, shape):
        if name not in outs:
            outs[name] = torch.empty(shape, dtype=torch.bfloat16, device=rt.device)
        return outs[name]

    def once():
        for m, f, xs in plan:
            rt.linear(xs[m.w_qkv.shape[1]], m.w_qkv, out("qkv", (tokens, m.w_qkv.shape[0])))
            rt.linear(xs[m.w_o.shape[1]], m.w_o, out("o", (tokens, m.w_o.shape[0])))
            rt.linear_swiglu(xs[f.w_gu.shape[1]], f.w_gu, f.group, out("act", (tokens, f.inter)))
            rt.linear(xs[f.w_down.shape[1]], f.w_down, out("down", (tokens, f.w_down.shape[0])))

    times = []
    for i in range(warmup + runs):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        once()
        e1.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(e0.elapsed_time(e1) / 1e3)
    return statistics.median(times), flops


def prefill_device(engine, tokens, runs=5, warmup=3):
    import numpy as np
    import torch
    from mlxforge_b200.engine.step import StepEntry
    runner, cache = engine.runner, engine.cache
    rng = np.random.default_rng(1)
    ids = rng.integers(0, engine.model.spec.vocab_size, size=tokens).tolist()
    times = []
    for i in range(warmup + runs):
        s = cache.open_sequence()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([StepEntry(s, ids, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        cache.close(s)
        if i >= warmup:
            times.append(e0.elapsed_time(e1) / 1e3)
    return statistics.median(times)


def decode_e2e(engine, batch, ctx, steps, warmup):
    """The same metric through the Python entry point: requests with host token ids
    in, generated ids out; every step copies its inputs from pinned host memory and
    reads the sampled ids back."""
    import numpy as np
    import torch
    import mlxforge_b200 as mf
    rng = np.random.default_rng(2)
    vocab = engine.model.spec.vocab_size
    # requests finish their prompts in different steps: every one gets room to decode through
    # the whole timed region, and is cancelled after it
    plen = ctx - (warmup + steps) - 1 - 2 * batch
    reqs = [engine.submit_ids(rng.integers(0, vocab, size=plen).tolist(), mf.GREEDY,
                              warmup + steps + 4 * batch + 64, eos_ids=[]) for _ in range(batch)]
    while any(len(r.output_ids) < 1 for r in reqs):          # prefill and first token, untimed
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    n0 = sum(len(r.output_ids) for r in reqs)
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    n1 = sum(len(r.output_ids) for r in reqs)
    h2d = engine.runner.last_meta_bytes
    assert all(not r.finished for r in reqs), "a request ended inside the timed region"
    for r in reqs:
        r.cancel()
    engine.run_until_idle()
    return (n1 - n0) / (t1 - t0), h2d, batch * 4 + 4      # the sampled ids and the kernels' status word


def serving_workload(engine, n_requests, lo, hi, out_tokens, seed=4):
    """The continuous-batching run of the reference's benchmark (bench/config.py:34-47 gives the
    load shapes; apps/mlxforge_cli.cpp:311-349 the protocol): `n_requests` requests with
    uniform-random prompt lengths in [lo, hi] submitted at once, `out_tokens` generated tokens
    each (EOS off), prompts run in portions beside decoding.  Host token ids in, ids out."""
    import numpy as np
    import torch
    import mlxforge_b200 as mf
    rng = np.random.default_rng(seed)
    vocab = engine.model.spec.vocab_size
    lens = rng.integers(lo, hi + 1, size=n_requests)
    prompts = [rng.integers(0, vocab, size=int(n)).tolist() for n in lens]
    torch.cuda.synchronize()
    steps_before = int(engine.metrics()["steps"])
    t0 = time.perf_counter()
    reqs = [engine.submit_ids(p, mf.GREEDY, out_tokens, eos_ids=[]) for p in prompts]
    first = [None] * n_requests
    while not engine.idle:
        engine.step()
        now = time.perf_counter()
        for i, r in enumerate(reqs):
            if first[i] is None and len(r.output_ids) > 0:
                first[i] = now
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    assert all(r.finish_reason == "length" for r in reqs), [r.finish_reason for r in reqs]
    ttft = sorted((f - t0) * 1e3 for f in first)
    gen = sum(len(r.output_ids) for r in reqs)
    m = engine.metrics()
    return {"seconds": round(t1 - t0, 3), "prompt_tokens": int(lens.sum()), "generated_tokens": gen,
            "tokens_per_s": round((int(lens.sum()) + gen) / (t1 - t0), 1), "generated_per_s": round(gen / (t1 - t0), 1),
            "ttft_ms_p50": round(ttft[len(ttft) // 2], 1), "ttft_ms_p99": round(ttft[min(len(ttft) - 1, int(0.99 * len(ttft)))], 1),
            "steps": int(m["steps"]) - steps_before, "preemptions": int(m["preemptions"]), "peak_running": int(m["peak_running"])}


def run_workload(args) -> int:
    """`--workload serving`: the Llama-3.2-3B shape, 64 requests with prompts of 128 to 4096
    tokens and 256 generated tokens each, portions of 512 beside decoding.  `--workload longctx`:
    the Llama-3.1-8B shape, 8 requests of 16,384 prompt tokens and 512 generated tokens each.
    Both print one JSON line; the first run on an engine also captures its CUDA graphs and
    sizes its buffers, so the load runs twice and both runs are reported."""
    import torch
    import mlxforge_b200 as mf
    from mlxforge_b200.config import config_from_json
    from mlxforge_b200.csrc import ops
    serving = args.workload == "serving"
    shape_key = args.shape if args.shape_given else ("3b" if serving else "8b")
    shape_name, shape = SHAPES[shape_key]
    layers = args.layers or shape["num_hidden_layers"]
    cfg_json = dict(shape, num_hidden_layers=layers)
    if serving:
        n, lo, hi, out, chunk, running = 64, 128, 4096, 256, 512, 64
    else:
        n, lo, hi, out, chunk, running = 8, 16384, 16384, 512, 2048, 8
    tmp = tempfile.mkdtemp(prefix="mlxforge_bench_")
    try:
        model_dir = mf.write_random_model(os.path.join(tmp, "model"), config_from_json(cfg_json), seed=0, dtype="bfloat16")
        engine = mf.Engine(model_spec=model_dir, dtype="bfloat16", kv_pool_tokens=n * (hi + out + 64), max_running=running,
                           token_budget=max(2048, chunk + running), prefill_chunk=chunk)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    clocks = ClockSampler()
    clocks.start()
    runs = [serving_workload(engine, n, lo, hi, out) for _ in range(2)]
    clk = clocks.stop()
    ops.check_kernel_status()
    print(json.dumps({
        "workload": args.workload, "model": f"{shape_name} shape", "layers": layers,
        "layers_of_named_config": shape["num_hidden_layers"], "requests": n, "prompt_tokens": [lo, hi],
        "generated_tokens_each": out, "prefill_chunk": chunk, "max_running": running, "dtype": "bf16",
        "data": "synthetic: seeded normal(0, 0.02) weights, seeded uniform token ids", "first_run": runs[0],
        "second_run": runs[1], "clocks": clk}))
    return 0


# ---------------------------------------------------------------------------- --workload notirax
# The Notirax design at sizes that resemble a real model's layers, beside the closest existing
# model (the Llama decoder) at equal size: the same width, heads, head size, layers and
# vocabulary, and a feed-forward as wide as the experts one token uses.
NOTIRAX_SIZES = {
    "s": dict(width=1024, heads=8, kv=2, dim=128, experts=32, top=4, ff=512, groups=4, keep=2, chunk=1024, layers=4,
              vocab=32768, streams=4, norm_groups=4, rank=64, conv=4),
    "m": dict(width=2048, heads=16, kv=4, dim=128, experts=64, top=6, ff=768, groups=8, keep=4, chunk=2048, layers=4,
              vocab=32768, streams=4, norm_groups=4, rank=128, conv=4),
}
FP32_TFLOPS_NOMINAL = 148 * 128 * 2 * 1.965e9 / 1e12      # FMA lanes x 2 x the maximum SM clock: no measured figure


def notirax_config(z):
    attn = {"type": "attention", "mixer": {"heads": z["heads"], "kv_heads": z["kv"], "dim": z["dim"], "vdim": z["dim"],
                                           "scale": z["dim"] ** -0.5, "softcap": 30.0, "mask": {"size": z["chunk"]}}}
    delta = {"type": "channel_delta", "mixer": {"heads": z["heads"], "kv_heads": z["heads"], "dim": z["dim"],
                                                "vdim": z["dim"], "conv": z["conv"], "decay_rank": z["rank"],
                                                "gate_rank": z["rank"]}}
    mlp = {"kind": "moe", "expert": {"ff": z["ff"], "limit": 7.0},
           "router": {"experts": z["experts"], "top": z["top"], "scale": 1.0,
                      "groups": {"count": z["groups"], "keep": z["keep"]}}}
    layers = [dict(delta if i % 2 == 0 else attn, mlp=mlp) for i in range(z["layers"])]
    return {"architecture": "Notirax", "vocab": z["vocab"], "width": z["width"], "streams": z["streams"],
            "norm": {"eps": 1e-6, "groups": z["norm_groups"]}, "layers": layers}


def llama_like(z):
    return dict(LLAMA_1B, num_hidden_layers=z["layers"], hidden_size=z["width"], num_attention_heads=z["heads"],
                num_key_value_heads=z["kv"], head_dim=z["dim"], intermediate_size=z["top"] * z["ff"],
                vocab_size=z["vocab"], rope_scaling=None)


class KernelTimes:
    """Records every call of the named launchers during one step, then times each recorded call
    alone: an event pair around the launch, the L2 flushed before it, the median of `reps`."""

    def __init__(self, names):
        from mlxforge_b200.csrc import ops
        self.ops, self.names, self.calls, self.saved = ops, names, [], {}

    def __enter__(self):
        import torch
        for n in self.names:
            # the library's grouped product is not one of this engine's launchers but stands among them
            owner = torch if n == "_grouped_mm" else self.ops
            if not hasattr(owner, n):
                continue
            fn = getattr(owner, n)
            self.saved[n] = (owner, fn)

            def rec(*a, _n=n, _fn=fn, **k):
                self.calls.append((_n, _fn, a, k))
                return _fn(*a, **k)
            setattr(owner, n, rec)
        return self

    def __exit__(self, *exc):
        for n, (owner, fn) in self.saved.items():
            setattr(owner, n, fn)

    def measure(self, reps=7):
        import torch
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        out = {}
        for n, fn, a, k in self.calls:
            ts = []
            for i in range(reps + 2):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn(*a, **k)
                e1.record()
                torch.cuda.synchronize()
                if i >= 2:
                    ts.append(e0.elapsed_time(e1) * 1e3)
            out.setdefault(n, []).append((statistics.median(ts), a, k))
        return out


def _nbytes(*ts):
    return sum(t.numel() * t.element_size() for t in ts if t is not None)


def kernel_work(name, a, k, info):
    """(bytes moved, tensor FLOPs, 32-bit FLOPs) that one call has to do, from its operands."""
    T, pairs, ctx_keys = info["tokens"], info["pairs"], info["ctx_keys"]
    if name == "hyper_update_norm":
        streams, delta, out, rows = a[0], a[1], a[9], (a[11] if len(a) > 11 else k.get("rows"))
        n = out.shape[0]
        s_bytes = n * streams.shape[1] * 4
        return (s_bytes * (2 if delta is not None and rows is None else 1) + _nbytes(out) + (n * out.shape[1] * delta.element_size() if delta is not None else 0), 0, 0)
    if name == "add_rmsnorm":
        resid, delta, out = a[0], a[1], a[4]
        n = out.shape[0]
        rows = a[5] if len(a) > 5 else k.get("rows")
        return (n * resid.shape[1] * 4 * (2 if delta is not None and rows is None else 1) + _nbytes(out) + (n * out.shape[1] * delta.element_size() if delta is not None else 0), 0, 0)
    if name == "attention_talking_tc":
        H, dim, vdim = a[11], a[13], a[14]
        return (0, 2.0 * pairs * H * (dim + vdim), 2.0 * pairs * H * H)
    if name == "attention_prefill":
        H, hd = a[11], a[13]
        return (0, 2.0 * pairs * H * 2 * hd, 0)
    if name == "attention_talking":
        n_kv, dim, vdim = a[9], a[10], a[11]
        return (ctx_keys * n_kv * (dim + vdim) * 2, 0, 0)
    if name == "attention_talking_decode":
        n_kv, dim, vdim = a[10], a[11], a[12]
        return (ctx_keys * n_kv * (dim + vdim) * 2, 0, 0)
    if name == "attention_decode":
        n_kv, hd = a[11], a[12]
        return (ctx_keys * n_kv * 2 * hd * 2, 0, 0)
    if name == "delta_recurrence":
        qkv, beta, ag, state, o, nh, dim, vdim = a[0], a[1], a[2], a[3], a[5], a[6], a[8], a[9]
        n_seqs = info["seqs"]
        return (_nbytes(qkv, beta, o) + ag.shape[0] * nh * dim * 4 + 2 * n_seqs * nh * dim * vdim * 4, 0,
                7.0 * T * nh * dim * vdim)
    if name in ("delta_prepare", "delta_gates", "delta_output", "biased_kv_store", "rope_kv_write", "moe_combine",
                "embed_positions", "embed", "swiglu"):
        return (_nbytes(*[t for t in a if hasattr(t, "numel") and t.dim() >= 2 and t.numel() < (1 << 28)]), 0, 0)
    if name == "moe_grouped_up":
        x, w_gu = a[0], a[1]
        return (0, 2.0 * T * a[6] * 2 * w_gu.shape[2] * x.shape[1], 0)
    if name == "moe_grouped_down":
        w_down = a[1]
        return (0, 2.0 * a[5] * a[6] * w_down.shape[1] * w_down.shape[2], 0)
    if name == "_grouped_mm":
        x, w = a[0], a[1]
        return (0, 2.0 * x.shape[0] * w.shape[1] * w.shape[2], 0)
    if name in ("moe_route", "moe_sort", "unary_act"):
        return (_nbytes(*[t for t in a if hasattr(t, "numel")]), 0, 0)
    if name == "mid_linear":
        x, w, out = a[0], a[1], a[2]
        return (_nbytes(x, w, out), 2.0 * x.shape[0] * w.shape[0] * w.shape[1], 0)
    if name in ("moe_gather_rows", "moe_activation"):
        return (_nbytes(*[t for t in a if hasattr(t, "numel") and t.dim() >= 2]), 0, 0)
    if name == "moe_rows":
        x, w_gu, ids = a[0], a[1], a[3]
        return (ids.numel() * 3 * w_gu.shape[2] * x.shape[1] * 2, 0, 0)
    if name == "add_rmsnorm_pair":
        resid, d1, d2, out1, out2 = a[0], a[1], a[2], a[6], a[7]
        rows = a[8] if len(a) > 8 else k.get("rows")
        n = out1.shape[0]
        moved = n * resid.shape[1] * 4 * (2 if (d1 is not None or d2 is not None) and rows is None else 1)
        return (moved + _nbytes(out1, out2) + sum(n * d.shape[1] * d.element_size() for d in (d1, d2) if d is not None), 0, 0)
    if name in ("attention_prefill_ex", "attention_decode_ex"):
        pre = name == "attention_prefill_ex"
        H, n_kv, hd, window, vd, in_k = (a[11], a[12], a[13], a[15], a[16], a[17]) if pre else \
            (a[10], a[11], a[12], a[14], a[16], a[17])
        keep = (a[18] if len(a) > 18 else k.get("keep_first", 0)) if window else 0
        if pre:
            seen = sum(min(p + 1, window + keep) if window else p + 1 for p in range(T))
            return (0, 2.0 * seen * H * (hd + vd), 0)
        seen = info["seqs"] * (min(info["ctx"], window + keep) if window else info["ctx"])
        return (seen * n_kv * (hd + (0 if in_k else vd)) * 2, 0, 0)
    if name in ("head_linear", "head_linear_mma"):
        w, n_tok = a[3], a[7]
        heads, n, kk = w.shape
        return (_nbytes(w) + n_tok * heads * (n + kk) * w.element_size(), 2.0 * n_tok * heads * n * kk, 0)
    if name == "retention_recurrence":
        qk, state, o, nh, dim, vdim = a[0], a[4], a[6], a[7], a[8], a[9]
        return (_nbytes(qk) + 4 * T * nh * vdim + T * nh * vdim * 2 + 2 * info["seqs"] * nh * dim * vdim * 4, 0,
                4.0 * T * nh * dim * vdim)
    if name in ("rope_store", "latent_prepare", "latent_query", "retention_prepare", "retention_output"):
        return (_nbytes(*[t for t in a if hasattr(t, "numel") and t.dim() >= 2 and t.numel() < (1 << 28)]), 0, 0)
    if name in ("gemm_bf16", "stream_linear"):
        x, w, out = a[0], a[1], a[2]
        return (_nbytes(x, w, out), 2.0 * x.shape[0] * w.shape[0] * w.shape[1], 0)
    if name == "conv_input":
        x, out = a[0], a[5]
        return (_nbytes(x, out), 0, 0)
    if name == "postnorm_add":
        x, y1, y2 = a[0], a[1], a[3]
        return (2 * _nbytes(x) + _nbytes(y1, y2), 0, 0)
    if name == "gdelta_recurrence":
        operands, state, o, nh, dim = a[0], a[5], a[7], a[8], a[9]
        return (_nbytes(operands, o) + 2 * T * nh * dim * 4 + 2 * info["seqs"] * nh * dim * dim * 4, 0,
                9.0 * T * nh * dim * dim)
    if name in ("qk_norm_rope", "rotate_rows", "gdelta_prepare", "delta_gates_ex"):
        return (_nbytes(*[t for t in a if hasattr(t, "numel") and t.dim() >= 2 and t.numel() < (1 << 28)]), 0, 0)
    return (0, 0, 0)


NOTIRAX_KERNELS = ("embed_positions", "hyper_update_norm", "biased_kv_store", "attention_talking", "attention_talking_tc",
                   "attention_talking_decode",
                   "delta_prepare", "delta_gates", "delta_recurrence", "delta_output", "moe_route", "moe_rows",
                   "moe_combine", "moe_sort", "moe_grouped_up", "moe_grouped_down", "moe_gather_rows", "moe_activation",
                   "_grouped_mm", "stream_linear", "gemm_bf16")
LLAMA_KERNELS = ("embed", "add_rmsnorm", "rope_kv_write", "attention_prefill", "attention_decode", "swiglu",
                 "stream_linear", "gemm_bf16")


def kernel_table(engine, names, tokens, batch, ctx, chunk, pk, extra=None):
    """Per kind of kernel: microseconds per call in a prefill of `tokens` tokens and in a decode step of
    `batch` sequences at `ctx`, and the fraction of the roofline (the slowest of bytes / HBM copy,
    tensor FLOPs / the library's bfloat16 product and 32-bit FLOPs / the nominal FMA rate)."""
    import numpy as np
    import torch
    from mlxforge_b200.engine.step import StepEntry
    runner, cache = engine.runner, engine.cache
    rng = np.random.default_rng(5)
    vocab = engine.model.spec.vocab_size
    table = {}

    def visible(n, first=0):
        return sum((p % chunk if chunk else p) + 1 for p in range(first, first + n))

    def collect(phase, entries, info):
        with KernelTimes(names) as kt:
            runner.step(entries)
            torch.cuda.synchronize()
        for n, calls in kt.measure().items():
            # the call whose time is the median of its kind stands for the kind, with its own work
            us, a, k = sorted(calls, key=lambda c: c[0])[len(calls) // 2]
            b, tf, ff = kernel_work(n, a, k, dict(info, **(extra or {})))
            roof = max(b / (pk["hbm_gbs"] * 1e9), tf / (pk["bf16_tflops"] * 1e12), ff / (FP32_TFLOPS_NOMINAL * 1e12)) * 1e6
            table[f"{phase}.{n}"] = {"us": round(us, 1), "calls": len(calls), "roof_us": round(roof, 2),
                                     "frac": round(roof / us, 3) if roof else None,
                                     "bound": None if not roof else ("hbm" if roof == b / (pk["hbm_gbs"] * 1e9) * 1e6 else
                                                                     "tensor" if roof == tf / (pk["bf16_tflops"] * 1e12) * 1e6 else "fp32")}

    s = cache.open_sequence()
    collect("prefill", [StepEntry(s, rng.integers(0, vocab, size=tokens).tolist(), [tokens - 1])],
            {"tokens": tokens, "pairs": visible(tokens), "ctx_keys": 0, "seqs": 1})
    cache.close(s)
    seqs = [cache.open_sequence() for _ in range(batch)]
    for q in seqs:
        cache.reserve([(q, ctx - 1)])
        cache.commit(q, ctx - 1)
    engine.runner.cuda_graphs, graphs = False, engine.runner.cuda_graphs
    try:
        collect("decode", [StepEntry(q, [int(rng.integers(0, vocab))], [0]) for q in seqs],
                {"tokens": batch, "pairs": 0, "ctx_keys": batch * visible(1, ctx - 1), "seqs": batch})
    finally:
        engine.runner.cuda_graphs = graphs
    for q in seqs:
        cache.close(q)
    return table


def run_notirax(args) -> int:
    import torch
    import mlxforge_b200 as mf
    from mlxforge_b200.config import config_from_json
    from mlxforge_b200.csrc import ops
    pk = peaks()
    out = {"workload": "notirax", "dtype": "bf16", "peaks": pk,
           "data": "synthetic: seeded random weights, seeded uniform token ids, random cache contents",
           "fp32_tflops_nominal": round(FP32_TFLOPS_NOMINAL, 1), "sizes": {}}
    clocks = ClockSampler()
    clocks.start()
    for key in ([args.size] if args.size else sorted(NOTIRAX_SIZES)):
        z = NOTIRAX_SIZES[key]
        res = {"size": z}
        for which, cfg_json, names in (("notirax", notirax_config(z), NOTIRAX_KERNELS),
                                       ("llama_equal_size", llama_like(z), LLAMA_KERNELS)):
            tmp = tempfile.mkdtemp(prefix="mlxforge_bench_")
            try:
                d = mf.write_random_model(os.path.join(tmp, "model"), config_from_json(cfg_json), seed=0, dtype="bfloat16")
                engine = mf.Engine(model_spec=d, dtype="bfloat16", kv_pool_tokens=(args.batch + 2) * (z["chunk"] + 2048 + 64),
                                   max_running=max(8, args.batch), token_budget=8192, prefill_chunk=2048)
            finally:
                shutil.rmtree(tmp, ignore_errors=True)
            for pool in engine.cache._k + engine.cache._v:
                pool.normal_(0.0, 1.0)
            ctx = z["chunk"]
            t_pre = prefill_device(engine, PREFILL_TOKENS, runs=3, warmup=3)
            sec, launches, _, _ = decode_device(engine, args.batch, ctx, args.steps, args.warmup)
            r = {"prefill_tokens": PREFILL_TOKENS, "prefill_ms": round(t_pre * 1e3, 3),
                 "prefill_tokens_per_s": round(PREFILL_TOKENS / t_pre, 1), "decode_batch": args.batch, "decode_context": ctx,
                 "decode_ms_per_step": round(sec * 1e3, 4), "decode_tokens_per_s": round(args.batch / sec, 1),
                 "decode_launches_per_step": launches, "graph_replays": engine.runner.graph_replays,
                 "weight_bytes_per_step": engine.model.weight_bytes()}
            if not args.skip_points:
                r["kernels"] = kernel_table(engine, names, PREFILL_TOKENS, args.batch, ctx,
                                            z["chunk"] if which == "notirax" else 0, pk)
            ops.check_kernel_status()
            res[which] = r
            del engine
            torch.cuda.empty_cache()
        out["sizes"][key] = res
    out["clocks"] = clocks.stop()
    print(json.dumps(out))
    return 0


# ---------------------------------------------------------------------------- --workload luzinex
# The Luzinex design at sizes that resemble a real model's layers, beside the closest existing model
# (the Llama decoder) at equal size: the same width, layers, vocabulary and feed-forward width, the
# heads and head size of its windowed attention layers.
LUZINEX_SIZES = {
    "s": dict(width=1024, layers=6, vocab=32768, ff=4096, heads=8, kv=2, dim=128, rot=64, window=1024, keep=4,
              l_heads=8, l_dim=64, l_rot=32, l_vdim=64, q_rank=384, kv_rank=128, r_heads=8, r_dim=128, r_vdim=128,
              context=4096),
    "m": dict(width=2048, layers=6, vocab=32768, ff=8192, heads=16, kv=4, dim=128, rot=64, window=2048, keep=4,
              l_heads=16, l_dim=64, l_rot=32, l_vdim=64, q_rank=768, kv_rank=192, r_heads=16, r_dim=128, r_vdim=128,
              context=4096),
}
LUZINEX_KERNELS = ("embed", "add_rmsnorm_pair", "rope_store", "latent_prepare", "latent_query", "head_linear", "head_linear_mma",
                   "attention_prefill_ex", "attention_decode_ex", "attention_generic_ex", "retention_prepare",
                   "retention_recurrence", "retention_chunked", "retention_output", "swiglu", "stream_linear", "gemm_bf16")


def luzinex_config(z):
    latent = {"heads": z["l_heads"], "dim": z["l_dim"], "rot_dim": z["l_rot"], "vdim": z["l_vdim"], "q_rank": z["q_rank"],
              "kv_rank": z["kv_rank"], "scale": (z["l_dim"] + z["l_rot"]) ** -0.5, "rot": {"base": 500000.0, "dims": z["l_rot"]}}
    attn = {"heads": z["heads"], "kv_heads": z["kv"], "dim": z["dim"], "vdim": z["dim"], "scale": z["dim"] ** -0.5,
            "rot": {"base": 50000.0, "dims": z["rot"]}, "mask": {"size": z["window"], "keep_first": z["keep"]}}
    ret = {"heads": z["r_heads"], "dim": z["r_dim"], "vdim": z["r_vdim"], "rot": {"base": 1000000.0, "dims": z["r_dim"]},
           "decay": [1.0 - 2.0 ** -(5 + 6.0 * h / z["r_heads"]) for h in range(z["r_heads"])]}
    mlp = {"kind": "dense", "ff": z["ff"]}
    layers = []
    for i in range(z["layers"]):
        kind = ("latent_attention", "attention", "retention")[i % 3]
        mixer = dict(latent, **({"kv_from": 0} if i >= 3 else {})) if kind == "latent_attention" else \
            dict(attn) if kind == "attention" else dict(ret)
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Luzinex", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "layers": layers}


def luzinex_llama_like(z):
    return dict(LLAMA_1B, num_hidden_layers=z["layers"], hidden_size=z["width"], num_attention_heads=z["heads"],
                num_key_value_heads=z["kv"], head_dim=z["dim"], intermediate_size=z["ff"], vocab_size=z["vocab"],
                rope_scaling=None, tie_word_embeddings=False)


def run_luzinex(args) -> int:
    import torch
    import mlxforge_b200 as mf
    from mlxforge_b200.config import config_from_json
    from mlxforge_b200.csrc import ops
    pk = peaks()
    out = {"workload": "luzinex", "dtype": "bf16", "peaks": pk,
           "data": "synthetic: seeded random weights, seeded uniform token ids, random cache contents",
           "fp32_tflops_nominal": round(FP32_TFLOPS_NOMINAL, 1), "sizes": {}}
    clocks = ClockSampler()
    clocks.start()
    for key in ([args.size] if args.size else sorted(LUZINEX_SIZES)):
        z = LUZINEX_SIZES[key]
        res = {"size": z}
        for which, cfg_json, names in (("luzinex", luzinex_config(z), LUZINEX_KERNELS),
                                       ("llama_equal_size", luzinex_llama_like(z), LLAMA_KERNELS)):
            tmp = tempfile.mkdtemp(prefix="mlxforge_bench_")
            try:
                d = mf.write_random_model(os.path.join(tmp, "model"), config_from_json(cfg_json), seed=0, dtype="bfloat16")
                engine = mf.Engine(model_spec=d, dtype="bfloat16", kv_pool_tokens=(args.batch + 2) * (z["context"] + 2048 + 64),
                                   max_running=max(8, args.batch), token_budget=8192, prefill_chunk=2048)
            finally:
                shutil.rmtree(tmp, ignore_errors=True)
            for pool in set(engine.cache._k + engine.cache._v):
                pool.normal_(0.0, 1.0)
            ctx = z["context"]
            t_pre = prefill_device(engine, PREFILL_TOKENS, runs=3, warmup=3)
            sec, launches, _, _ = decode_device(engine, args.batch, ctx, args.steps, args.warmup)
            r = {"prefill_tokens": PREFILL_TOKENS, "prefill_ms": round(t_pre * 1e3, 3),
                 "prefill_tokens_per_s": round(PREFILL_TOKENS / t_pre, 1), "decode_batch": args.batch, "decode_context": ctx,
                 "decode_ms_per_step": round(sec * 1e3, 4), "decode_tokens_per_s": round(args.batch / sec, 1),
                 "decode_launches_per_step": launches, "graph_replays": engine.runner.graph_replays,
                 "weight_bytes_per_step": engine.model.weight_bytes()}
            if not args.skip_points:
                r["kernels"] = kernel_table(engine, names, PREFILL_TOKENS, args.batch, ctx, 0, pk, extra={"ctx": ctx})
            ops.check_kernel_status()
            res[which] = r
            del engine
            torch.cuda.empty_cache()
        out["sizes"][key] = res
    out["clocks"] = clocks.stop()
    print(json.dumps(out))
    return 0


# ---------------------------------------------------------------------------- --workload rabapel
# The Rabapel design at sizes that resemble a real model's layers, beside the closest existing model at
# equal size: a Luzinex decoder made of latent-attention layers only (the same width, layers, vocabulary,
# heads, head sizes and latent rank; its queries through a latent of their own, no window, a gate per
# channel), with gated feed-forwards of the dense layers' parameter count.  Rabapel's layers alternate a
# dense squared-rectifier feed-forward and a mixture with identity experts and a gated shared expert; the
# mixture's kernels are those of the Notirax design (--workload notirax lists them at its sizes).
RABAPEL_SIZES = {
    "s": dict(width=1024, layers=6, vocab=32768, ff=4096, heads=8, dim=64, rot=32, vdim=64, kv_rank=128, q_rank=384,
              window=1024, experts=16, identity=2, top=4, expert_ff=512, shared_ff=1024, context=4096),
    "m": dict(width=2048, layers=6, vocab=32768, ff=8192, heads=16, dim=64, rot=32, vdim=64, kv_rank=192, q_rank=768,
              window=2048, experts=32, identity=4, top=6, expert_ff=768, shared_ff=2048, context=4096),
}
RABAPEL_KERNELS = ("embed", "add_rmsnorm_pair", "latent_prepare", "latent_query", "head_linear", "head_linear_mma",
                   "attention_prefill_ex", "attention_decode_ex", "attention_generic_ex", "moe_route", "moe_rows",
                   "moe_combine", "moe_sort", "moe_grouped_up", "moe_grouped_down", "moe_gather_rows", "moe_activation",
                   "_grouped_mm", "swiglu", "unary_act", "mid_linear", "stream_linear", "gemm_bf16")


def rabapel_config(z):
    mixer = {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot"], "vdim": z["vdim"], "kv_rank": z["kv_rank"],
             "scale": (z["dim"] + z["rot"]) ** -0.5, "mask": {"size": z["window"]},
             "rot": {"base": 500000.0, "dims": z["rot"],
                     "scaling": {"factor": 8.0, "original": z["context"] // 8, "fast": 32.0, "slow": 1.0}}}
    dense = {"kind": "dense", "ff": z["ff"]}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "shared": {"ff": z["shared_ff"]},
           "router": {"experts": z["experts"], "identity": z["identity"], "top": z["top"]}}
    return {"architecture": "Rabapel", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6},
            "embedding": {"scale": 0.5},
            "layers": [{"type": "latent_attention", "mixer": dict(mixer), "mlp": dense if i % 2 == 0 else moe}
                       for i in range(z["layers"])]}


def rabapel_luzinex_like(z):
    latent = {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot"], "vdim": z["vdim"], "q_rank": z["q_rank"],
              "kv_rank": z["kv_rank"], "scale": (z["dim"] + z["rot"]) ** -0.5, "rot": {"base": 500000.0, "dims": z["rot"]}}
    # a gated feed-forward has three matrices where the squared-rectifier one has two
    mlp = {"kind": "dense", "ff": z["ff"] * 2 // 3 // 128 * 128}
    return {"architecture": "Luzinex", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5},
            "layers": [{"type": "latent_attention", "mixer": dict(latent), "mlp": mlp} for _ in range(z["layers"])]}


def run_rabapel(args) -> int:
    import torch
    import mlxforge_b200 as mf
    from mlxforge_b200.config import config_from_json
    from mlxforge_b200.csrc import ops
    pk = peaks()
    out = {"workload": "rabapel", "dtype": "bf16", "peaks": pk,
           "data": "synthetic: seeded random weights, seeded uniform token ids, random cache contents",
           "fp32_tflops_nominal": round(FP32_TFLOPS_NOMINAL, 1), "sizes": {}}
    sampled = []
    for key in ([args.size] if args.size else sorted(RABAPEL_SIZES)):
        z = RABAPEL_SIZES[key]
        res = {"size": z}
        for which, cfg_json, names in (("rabapel", rabapel_config(z), RABAPEL_KERNELS),
                                       ("luzinex_latent_equal_size", rabapel_luzinex_like(z), LUZINEX_KERNELS)):
            tmp = tempfile.mkdtemp(prefix="mlxforge_bench_")
            try:
                d = mf.write_random_model(os.path.join(tmp, "model"), config_from_json(cfg_json), seed=0, dtype="bfloat16")
                engine = mf.Engine(model_spec=d, dtype="bfloat16", kv_pool_tokens=(args.batch + 2) * (z["context"] + 2048 + 64),
                                   max_running=max(8, args.batch), token_budget=8192, prefill_chunk=2048)
            finally:
                shutil.rmtree(tmp, ignore_errors=True)
            for pool in set(engine.cache._k + engine.cache._v):
                pool.normal_(0.0, 1.0)
            ctx = z["context"]
            # clocks while the device works: writing and loading a model is host time at idle clocks
            clocks = ClockSampler()
            clocks.start()
            t_pre = prefill_device(engine, PREFILL_TOKENS, runs=3, warmup=3)
            sec, launches, _, _ = decode_device(engine, args.batch, ctx, args.steps, args.warmup)
            r = {"prefill_tokens": PREFILL_TOKENS, "prefill_ms": round(t_pre * 1e3, 3),
                 "prefill_tokens_per_s": round(PREFILL_TOKENS / t_pre, 1), "decode_batch": args.batch, "decode_context": ctx,
                 "decode_ms_per_step": round(sec * 1e3, 4), "decode_tokens_per_s": round(args.batch / sec, 1),
                 "decode_launches_per_step": launches, "graph_replays": engine.runner.graph_replays,
                 "weight_bytes_per_step": engine.model.weight_bytes()}
            if not args.skip_points:
                r["kernels"] = kernel_table(engine, names, PREFILL_TOKENS, args.batch, ctx, 0, pk, extra={"ctx": ctx})
            r["clocks"] = clocks.stop()
            sampled.append(r["clocks"])
            ops.check_kernel_status()
            res[which] = r
            del engine
            torch.cuda.empty_cache()
        out["sizes"][key] = res
    seen = [c for c in sampled if c["sm_mhz"] is not None]
    out["clocks"] = {"sm_mhz": min(c["sm_mhz"] for c in seen) if seen else None,
                     "sm_max_mhz": max(c["sm_max_mhz"] for c in seen) if seen else None,
                     "reasons": sorted({x for c in seen for x in c["reasons"]})}
    print(json.dumps(out))
    return 0


# ---------------------------------------------------------------------------- --workload ledinex
# The Ledinex design at sizes that resemble a real model's layers, beside the closest existing model at equal
# size: a Notirax decoder (attention, a gated delta rule and a mixture of experts, like it) with the same width,
# layers, vocabulary, attention heads and head size, delta heads, experts and experts' width, one residual
# stream and one norm group.  Ledinex's layers are parallel_2, delta, parallel, delta, each with a mixture of
# squared-rectifier experts and a shared expert.
LEDINEX_SIZES = {
    "s": dict(width=1024, layers=4, vocab=32768, heads=8, kv=2, dim=128, window=1024, r_heads=8, r_dim=64, rank=64,
              l_heads=8, l_dim=64, l_vdim=128, d_heads=8, d_dim=128, conv=4, taps=3, experts=32, top=4, ff=512, shared_ff=1024,
              context=4096),
    "m": dict(width=2048, layers=4, vocab=32768, heads=16, kv=4, dim=128, window=2048, r_heads=16, r_dim=64, rank=64,
              l_heads=16, l_dim=64, l_vdim=128, d_heads=16, d_dim=128, conv=4, taps=3, experts=64, top=6, ff=768, shared_ff=2048,
              context=4096),
}
LEDINEX_KERNELS = ("embed", "conv_input", "postnorm_add", "qk_norm_rope", "rotate_rows", "attention_prefill_ex",
                   "attention_decode_ex", "attention_generic_ex", "retention_prepare", "retention_recurrence",
                   "retention_output", "gdelta_prepare", "gdelta_recurrence", "delta_gates_ex", "delta_prepare",
                   "delta_recurrence", "delta_output", "moe_route", "moe_rows", "moe_combine", "moe_sort",
                   "moe_grouped_up", "moe_grouped_down", "moe_gather_rows", "_grouped_mm", "unary_act", "add_rmsnorm",
                   "stream_linear", "gemm_bf16")


def ledinex_config(z):
    yarn = {"factor": 8.0, "original": z["context"] // 8, "fast": 32.0, "slow": 1.0}
    left2 = {"heads": z["heads"], "kv_heads": z["kv"], "dim": z["dim"], "vdim": z["dim"], "scale": z["dim"] ** -0.5,
             "mask": {"size": z["window"]}, "rot": {"base": 10000.0, "dims": z["dim"] // 2, "scaling": yarn}}
    left1 = {"heads": z["heads"], "kv_heads": z["kv"], "dim": z["dim"], "vdim": z["dim"], "scale": z["dim"] ** -0.5,
             "softcap": 50.0, "rot": {"base": 250000.0, "dims": z["dim"], "scaling": {"factor": 4.0}}}
    par2 = {"type": "parallel_2", "mixer": {"left": left2, "right": {"heads": z["r_heads"], "dim": z["r_dim"],
                                                                     "decay_rank": z["rank"]},
                                            "left_scale": 0.8, "right_scale": 0.9}}
    par = {"type": "parallel", "mixer": {"left": left1, "right": {"heads": z["l_heads"], "dim": z["l_dim"], "vdim": z["l_vdim"],
                                                                  "decay": [1.0 - 2.0 ** -(2 + i % 8) for i in range(z["l_heads"])]},
                                         "left_scale": 0.8, "right_scale": 0.9}}
    delta = {"type": "delta", "mixer": {"heads": z["d_heads"], "kv_heads": z["d_heads"], "dim": z["d_dim"], "vdim": z["d_dim"],
                                        "conv": z["conv"]}}
    mlp = {"kind": "moe", "expert": {"ff": z["ff"]}, "router": {"experts": z["experts"], "top": z["top"]},
           "shared": {"ff": z["shared_ff"]}}
    order = [par2, delta, par, delta]
    return {"architecture": "Ledinex", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5},
            "embedding": {"scale": 16.0}, "logit_scale": 2.0, "canon": {"taps": z["taps"]},
            "layers": [dict(order[i % 4], mlp=mlp) for i in range(z["layers"])]}


def ledinex_notirax_like(z):
    attn = {"type": "attention", "mixer": {"heads": z["heads"], "kv_heads": z["kv"], "dim": z["dim"], "vdim": z["dim"],
                                           "scale": z["dim"] ** -0.5, "softcap": 50.0, "mask": {"size": z["window"]}}}
    delta = {"type": "channel_delta", "mixer": {"heads": z["d_heads"], "kv_heads": z["d_heads"], "dim": z["d_dim"],
                                                "vdim": z["d_dim"], "conv": z["conv"], "decay_rank": z["rank"],
                                                "gate_rank": z["rank"]}}
    mlp = {"kind": "moe", "expert": {"ff": z["ff"], "limit": 7.0}, "router": {"experts": z["experts"], "top": z["top"], "scale": 1.0}}
    return {"architecture": "Notirax", "vocab": z["vocab"], "width": z["width"], "streams": 1,
            "norm": {"eps": 1e-6, "groups": 1},
            "layers": [dict(attn if i % 2 == 0 else delta, mlp=mlp) for i in range(z["layers"])]}


def run_ledinex(args) -> int:
    import torch
    import mlxforge_b200 as mf
    from mlxforge_b200.config import config_from_json
    from mlxforge_b200.csrc import ops
    pk = peaks()
    out = {"workload": "ledinex", "dtype": "bf16", "peaks": pk,
           "data": "synthetic: seeded random weights, seeded uniform token ids, random cache contents",
           "fp32_tflops_nominal": round(FP32_TFLOPS_NOMINAL, 1), "sizes": {}}
    sampled = []
    for key in ([args.size] if args.size else sorted(LEDINEX_SIZES)):
        z = LEDINEX_SIZES[key]
        res = {"size": z}
        for which, cfg_json, names, chunk in (("ledinex", ledinex_config(z), LEDINEX_KERNELS, 0),
                                              ("notirax_equal_size", ledinex_notirax_like(z), NOTIRAX_KERNELS, z["window"])):
            tmp = tempfile.mkdtemp(prefix="mlxforge_bench_")
            try:
                d = mf.write_random_model(os.path.join(tmp, "model"), config_from_json(cfg_json), seed=0, dtype="bfloat16")
                engine = mf.Engine(model_spec=d, dtype="bfloat16", kv_pool_tokens=(args.batch + 2) * (z["context"] + 2048 + 64),
                                   max_running=max(8, args.batch), token_budget=8192, prefill_chunk=2048)
            finally:
                shutil.rmtree(tmp, ignore_errors=True)
            for pool in set(engine.cache._k + engine.cache._v):
                pool.normal_(0.0, 1.0)
            ctx = z["context"]
            clocks = ClockSampler()
            clocks.start()
            t_pre = prefill_device(engine, PREFILL_TOKENS, runs=3, warmup=3)
            sec, launches, _, _ = decode_device(engine, args.batch, ctx, args.steps, args.warmup)
            r = {"prefill_tokens": PREFILL_TOKENS, "prefill_ms": round(t_pre * 1e3, 3),
                 "prefill_tokens_per_s": round(PREFILL_TOKENS / t_pre, 1), "decode_batch": args.batch, "decode_context": ctx,
                 "decode_ms_per_step": round(sec * 1e3, 4), "decode_tokens_per_s": round(args.batch / sec, 1),
                 "decode_launches_per_step": launches, "graph_replays": engine.runner.graph_replays,
                 "weight_bytes_per_step": engine.model.weight_bytes()}
            if not args.skip_points:
                r["kernels"] = kernel_table(engine, names, PREFILL_TOKENS, args.batch, ctx, chunk, pk, extra={"ctx": ctx})
            r["clocks"] = clocks.stop()
            sampled.append(r["clocks"])
            ops.check_kernel_status()
            res[which] = r
            del engine
            torch.cuda.empty_cache()
        out["sizes"][key] = res
    seen = [c for c in sampled if c["sm_mhz"] is not None]
    out["clocks"] = {"sm_mhz": min(c["sm_mhz"] for c in seen) if seen else None,
                     "sm_max_mhz": max(c["sm_max_mhz"] for c in seen) if seen else None,
                     "reasons": sorted({x for c in seen for x in c["reasons"]})}
    print(json.dumps(out))
    return 0


# Kinds of launches that `--without` leaves out of a decode step, to see what each costs inside it.
LEFT_OUT = ("norms", "rotation", "attention", "qkv", "o", "gate_up", "down", "head", "products")


def leave_out(kind: str, shape: dict) -> None:
    """Replace the launcher of one kind of kernel by nothing (the step's numbers are then wrong and
    only its time means something)."""
    from mlxforge_b200.csrc import ops
    hidden, inter = shape["hidden_size"], shape["intermediate_size"]
    qkv_rows = (shape["num_attention_heads"] + 2 * shape["num_key_value_heads"]) * shape["head_dim"]
    stream = ops.stream_linear

    def nothing(*a, **k):
        return None

    def products(pred):
        def f(x, w, out, swiglu=False):
            return None if pred(w, swiglu) else stream(x, w, out, swiglu=swiglu)
        return f

    if kind == "norms":
        ops.add_rmsnorm = nothing
    elif kind == "rotation":
        ops.rope_kv_write = nothing
    elif kind == "attention":
        ops.attention_decode = nothing
    elif kind == "products":
        ops.stream_linear = nothing
    else:
        pred = {"qkv": lambda w, s: not s and tuple(w.shape) == (qkv_rows, hidden),
                "o": lambda w, s: not s and tuple(w.shape) == (hidden, shape["num_attention_heads"] * shape["head_dim"])
                and tuple(w.shape) != (qkv_rows, hidden),
                "gate_up": lambda w, s: s,
                "down": lambda w, s: not s and tuple(w.shape) == (hidden, inter),
                "head": lambda w, s: w.shape[0] == shape["vocab_size"]}[kind]
        ops.stream_linear = products(pred)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default=None, choices=sorted(SHAPES), help="layer sizes (default: the 1B shape)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (0: all)")
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch")
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="decode / prefill: run just that part and print a short line (for profiling small cases)")
    ap.add_argument("--without", default=None, choices=sorted(LEFT_OUT),
                    help="with --only decode: time the step with the launches of one kind left out (its results are "
                         "wrong; the difference to the full step is what that kind costs inside the step)")
    ap.add_argument("--workload", default="headline", choices=["headline", "serving", "longctx", "notirax", "luzinex", "rabapel", "ledinex"],
                    help="serving: 64 requests on the 3B shape; longctx: 8 x 16,384 tokens on the 8B shape; notirax / "
                         "luzinex: prefill and decode of that design beside the Llama decoder at equal size, per kernel; "
                         "rabapel: the same beside a Luzinex decoder of latent-attention layers at equal size; "
                         "ledinex: the same beside a Notirax decoder at equal size")
    ap.add_argument("--size", default=None, choices=sorted(set(NOTIRAX_SIZES) | set(LUZINEX_SIZES) | set(RABAPEL_SIZES)),
                    help="with --workload notirax, luzinex, rabapel or ledinex: one size only")
    args = ap.parse_args()
    args.shape_given = args.shape is not None
    args.shape = args.shape or "1b"

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"unavailable": f"this engine runs on one GPU; --gpus {args.gpus} is not supported"}))
        return 2
    args.warmup = max(args.warmup, 3)
    if args.workload == "notirax":
        return run_notirax(args)
    if args.workload == "luzinex":
        return run_luzinex(args)
    if args.workload == "rabapel":
        return run_rabapel(args)
    if args.workload == "ledinex":
        return run_ledinex(args)
    if args.workload != "headline":
        return run_workload(args)

    import torch
    import mlxforge_b200 as mf
    from mlxforge_b200.config import config_from_json

    shape_name, shape = SHAPES[args.shape]
    args.layers = args.layers or shape["num_hidden_layers"]
    cfg_json = dict(shape, num_hidden_layers=args.layers)
    tmp = tempfile.mkdtemp(prefix="mlxforge_bench_")
    try:
        t0 = time.time()
        model_dir = mf.write_random_model(os.path.join(tmp, f"llama_{args.shape}_random"), config_from_json(cfg_json), seed=0,
                                          dtype="bfloat16")
        ctx = args.context
        pool_seqs = 64 if args.only == "all" and not args.skip_points else max(args.batch, 1)
        engine = mf.Engine(model_spec=model_dir, dtype="bfloat16", kv_pool_tokens=pool_seqs * (ctx + 64),
                           max_running=64, token_budget=8192, prefill_chunk=2048)
        print(f"[bench] model written and loaded in {time.time() - t0:.0f}s", file=sys.stderr, flush=True)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    # the synthetic cache: random keys and values everywhere (reading zeros is as slow, but keep it honest)
    for pool in engine.cache._k + engine.cache._v:
        pool.normal_(0.0, 1.0)

    pk = peaks()
    weight_bytes = engine.model.weight_bytes()
    kv_per_token = engine.model.cache_layout.bytes_per_token(2)

    if args.only == "prefill":
        t_pre = prefill_device(engine, PREFILL_TOKENS, runs=max(1, args.steps), warmup=args.warmup)
        print(json.dumps({"only": "prefill", "shape": args.shape, "tokens": PREFILL_TOKENS, "ms": round(t_pre * 1e3, 3),
                          "layers": args.layers}))
        return 0
    BATCH_ = args.batch
    if args.without:
        if args.only != "decode":
            print("--without goes with --only decode", file=sys.stderr)
            return 2
        leave_out(args.without, shape)
    clocks = ClockSampler()
    clocks.start()
    sec, launches, kv_tokens, pieces = decode_device(engine, BATCH_, ctx, args.steps, args.warmup)
    clk = clocks.stop()
    value = BATCH_ / sec
    bytes_step = weight_bytes + kv_tokens * kv_per_token
    achieved = bytes_step / sec / 1e9
    if args.only == "decode":
        line = {"only": "decode", "shape": args.shape, "batch": BATCH_, "context": ctx, "layers": args.layers,
                "ms_per_step": round(sec * 1e3, 4), "launches_per_step": launches, "gbs": round(achieved, 1)}
        if args.without:
            line = dict(line, without=args.without, gbs=None, note="a kind of kernel was left out: a timing, not a result")
        print(json.dumps(line))
        return 0

    # the other batch sizes the metric names, at the headline context and at the 1024 tokens its
    # decode line names; each with the fraction of the HBM peak that its bytes over its time are
    points, point_fracs = {}, {}
    if not args.skip_points:
        for b, c in ((1, ctx), (64, ctx), (1, 1024), (8, 1024), (64, 1024)):
            s_b, _, kv_b, _ = decode_device(engine, b, c, max(8, args.steps // 2), args.warmup, seed=b)
            name = f"decode_b{b}" if c == ctx else f"decode_b{b}_ctx{c}"
            points[name] = round(b / s_b, 1)
            point_fracs[name] = round((weight_bytes + kv_b * kv_per_token) / s_b / 1e9 / pk["hbm_gbs"], 4)

    t_pre = prefill_device(engine, PREFILL_TOKENS)
    t_gemm, gemm_flops = prefill_products_device(engine, PREFILL_TOKENS)
    c = cfg_json
    L, H, I, V = c["num_hidden_layers"], c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    nh, nkv, hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    mat = L * (H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * I)
    T = PREFILL_TOKENS
    flops = 2.0 * T * mat + 2.0 * V * H + L * 2.0 * T * T * hd * nh     # products + one head row + causal attention
    # the whole prefill is timed alone between synchronisations: the burst peak is its divisor
    prefill = {"value": round(T / t_pre, 1), "tokens": T, "ms": round(t_pre * 1e3, 3),
               "frac": round(flops / t_pre / (pk["bf16_tflops"] * 1e12), 4),
               "frac_of_sustained": round(flops / t_pre / (pk["bf16_tflops_sustained"] * 1e12), 4),
               "products_ms": round(t_gemm * 1e3, 3),
               "products_frac": round(gemm_flops / t_gemm / (pk["bf16_tflops"] * 1e12), 4)}

    e2e_value, h2d, d2h = decode_e2e(engine, BATCH_, ctx, args.steps, args.warmup)
    # what the Python host costs at the other batch sizes, and what launching a step before the tokens of
    # the one before are on the host is worth: the same metric through the entry point
    e2e_points = {}
    if not args.skip_points:
        half = max(8, args.steps // 2)
        e2e_points["decode_b1"] = round(decode_e2e(engine, 1, ctx, half, args.warmup)[0], 1)
        e2e_points["decode_b64_ctx1024"] = round(decode_e2e(engine, 64, 1024, half, args.warmup)[0], 1)
        engine.pipeline = False
        try:
            e2e_points["decode_b8_unpipelined"] = round(decode_e2e(engine, BATCH_, ctx, half, args.warmup)[0], 1)
            e2e_points["decode_b1_unpipelined"] = round(decode_e2e(engine, 1, ctx, half, args.warmup)[0], 1)
        finally:
            engine.pipeline = True

    line = {
        "metric": f"decode tok/s @ batch {BATCH_} ({shape_name} bf16)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded normal(0, 0.02) weights, seeded uniform token ids, random cache contents",
        "config": {
            "model": f"{shape_name} shape (LlamaForCausalLM)", "layers": L,
            "layers_of_named_config": shape["num_hidden_layers"],
            "hidden": H, "heads": nh, "kv_heads": nkv, "head_dim": hd, "intermediate": I, "vocab": V,
            "global_batch": BATCH_, "seq_len": ctx, "context_len": ctx, "kv_block": engine.cache.page_size,
            "prefill_tokens": T, "parallelism": "single GPU",
            "l2": "working set per step (weights + live cache) exceeds L2 many times; no flush needed",
            "peaks": pk["source"],
        },
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(round(launches * args.steps)),
        "clocks": clk,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "point_fracs": point_fracs,
        "e2e_points": e2e_points,
        "ms_per_step_pieces": {"median": round(statistics.median(pieces), 4), "min": round(min(pieces), 4),
                               "max": round(max(pieces), 4), "pieces": len(pieces)},
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
