#!/usr/bin/env python3
"""Benchmark of models_b200 on one B200: decode tokens per second of Llama 3.2 1B (bfloat16, random
weights, synthetic token ids), with prefill and roofline figures on the same JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--model 1b|3b|8b] [--batch B] [--layers L] [--impl ours|reference]

A "step" is one decode step of the whole batch.  `value` is device-timed (CUDA events around K
steps); `e2e` is the same rate through the Python entry point (`generate_batch`: host token ids in,
host token ids out, every step's indices copied to the device and its sampled ids copied back).
Each decode step reads about 2.5 GB of weights, far more than the 126 MB L2, so successive steps
do not find their inputs in the cache.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: Llama 3.2 1B
LLAMA_3_2_1B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 16,
    "hidden_size": 2048,
    "num_attention_heads": 32,
    "num_key_value_heads": 8,
    "head_dim": 64,
    "intermediate_size": 8192,
    "vocab_size": 128256,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True,
    "max_position_embeddings": 131072,
    "hidden_act": "silu",
}
CONTEXT = 4096
PROMPT_TOKENS = 512
PREFILL_TOKENS = 2048

# The other two workloads of the baseline file (--model 3b / 8b); the default run is the 1B one.
LLAMA_3_2_3B = dict(LLAMA_3_2_1B, num_hidden_layers=28, hidden_size=3072, num_attention_heads=24, num_key_value_heads=8,
                    head_dim=128, intermediate_size=8192)
LLAMA_3_1_8B = dict(LLAMA_3_2_1B, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                    head_dim=128, intermediate_size=14336, tie_word_embeddings=False,
                    rope_scaling=dict(LLAMA_3_2_1B["rope_scaling"], factor=8.0))
WORKLOADS = {
    # prompt: a length, or (shortest, longest) for unequal prompts; context: positions per sequence the cache is sized for
    "1b": {"config": LLAMA_3_2_1B, "name": "Llama 3.2 1B (LlamaForCausalLM)", "batch": 8, "prompt": PROMPT_TOKENS,
           "context": CONTEXT, "steps": 256, "prefill": PREFILL_TOKENS, "points": (1, 64)},
    "3b": {"config": LLAMA_3_2_3B, "name": "Llama 3.2 3B (LlamaForCausalLM)", "batch": 16, "prompt": (128, 2048),
           "context": 2048 + 192, "steps": 128, "prefill": PREFILL_TOKENS, "points": ()},
    "8b": {"config": LLAMA_3_1_8B, "name": "Llama 3.1 8B-shaped (LlamaForCausalLM)", "batch": 64, "prompt": 1024,
           "context": 1024 + 320, "steps": 256, "prefill": 16384, "points": ()},
}

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    """The roofline denominators: the driver's measured copy bandwidth and cuBLAS bf16 throughput (burst) when
    MEASURED_PEAKS.json is there, else the stated fallback figures."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")

    def number(raw, names, scale=1.0):
        for name in names:
            value = raw.get(name)
            if isinstance(value, dict):
                value = value.get("value", value.get("measured"))
            if isinstance(value, (int, float)) and value > 0:
                return float(value) * scale
        return None

    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            hbm = number(raw, ("hbm_gbs", "hbm_gb_s", "hbm_gbps")) or number(raw, ("hbm_tbs", "hbm_tb_s"), 1000.0)
            bf16 = number(raw, ("bf16_tflops", "bf16_tflops_burst")) or number(raw, ("bf16_pflops",), 1000.0)
            if hbm and bf16:
                return {"hbm_gbs": hbm, "bf16_tflops": bf16, "source": "measured"}
        except (OSError, ValueError, TypeError, AttributeError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.process = None
        self.skip = 0

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "25"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.process = None
            return
        # the tool takes a moment to come up; the timed region starts once it is sampling
        deadline = time.perf_counter() + 3.0
        while time.perf_counter() < deadline and os.path.getsize(self.file.name) == 0:
            time.sleep(0.02)
        self.skip = os.path.getsize(self.file.name)  # what it printed before the timed region

    def stop(self):
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
        self.file.flush()
        self.file.seek(self.skip)
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                max_clock = float(parts[1])
            except ValueError:
                continue
            for name, value in zip(names, parts[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def matmul_params(c, layers):
    q, kv = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    d, i = c["hidden_size"], c["intermediate_size"]
    per_layer = d * (q + 2 * kv) + q * d + 3 * d * i
    return layers * per_layer, c["vocab_size"] * d


def decode_bytes(c, layers, kv_tokens_total):
    """Bytes a decode step has to read: every weight once (layers, norms, output matrix), and the
    keys and values of the live requests."""
    layer_params, head_params = matmul_params(c, layers)
    norms = (2 * layers + 1) * c["hidden_size"]
    weights = 2 * (layer_params + head_params) + 4 * norms
    kv = kv_tokens_total * layers * 2 * c["num_key_value_heads"] * c["head_dim"] * 2
    return weights + kv


def prefill_flops(c, layers, tokens):
    layer_params, head_params = matmul_params(c, layers)
    gemm = 2 * tokens * layer_params + 2 * head_params  # the output matrix runs on one row
    attention = layers * 4 * c["num_attention_heads"] * c["head_dim"] * tokens * tokens / 2
    return gemm + attention


def make_model(config, max_batch, context=CONTEXT):
    import models_b200

    return models_b200.load_model(config=config, seed=0, dtype="bfloat16", max_batch=max_batch, context=context)


def random_prompts(n, length, vocab, seed):
    """n prompts of `length` tokens each, or of lengths drawn from (shortest, longest)."""
    import numpy as np

    rng = np.random.default_rng(seed)
    lengths = [length] * n if isinstance(length, int) else [int(x) for x in rng.integers(length[0], length[1] + 1, size=n)]
    return [[int(t) for t in rng.integers(0, vocab, size=m)] for m in lengths]


def device_decode(model, batch, steps, warmup, sample_clocks=False, prompt=PROMPT_TOKENS):
    """K decode steps of `batch` sequences after their prompts (512 tokens each in the default run), greedy, timed on the device.
    As in generation, a step is queued with the ids of the step before it still on the device, and
    the host reads every step's ids while the next step runs."""
    import torch

    from models_b200 import SamplingOptions
    from models_b200.engine.stepper import EngineStepper
    from models_b200.kernels import ops
    from models_b200.sampling.sampler import RequestSampling

    engine = model.engine
    vocab = engine.spec.vocab_size
    prompts = random_prompts(batch, prompt, vocab, 1)
    stepper = EngineStepper(engine)
    greedy = [RequestSampling(SamplingOptions(temperature=0.0), p) for p in prompts]
    rows = list(range(batch))
    slots = [stepper.open_slot() for _ in range(batch)]
    pending = stepper.sample_start(stepper.prefill(slots, prompts), greedy)
    for _ in range(warmup):
        logits = stepper.decode_pending(slots, pending, rows)
        pending.result()
        pending = stepper.sample_start(logits, greedy)
    graphs = engine.decode_graphs
    if graphs is not None and batch <= graphs.max_batch:
        # part of the warm-up: the captures of every class of context length that the timed steps will meet (a
        # sequence that crosses such a boundary would otherwise pay for a capture inside the timed region)
        longest = max(engine.length(s) for s in slots)
        for kv in range(longest + 1, longest + steps + 2):
            graphs.prepare(graphs.rung(batch), kv)
    sampler = ClockSampler() if sample_clocks else None
    if sampler:
        sampler.start()
    kv_total = 0
    launches_before = ops.launch_count()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]  # one after every step, on the step's stream
    torch.cuda.synchronize()
    marks[0].record()
    for step in range(steps):
        kv_total += sum(engine.length(s) + 1 for s in slots)
        logits = stepper.decode_pending(slots, pending, rows)
        pending.result()
        pending = stepper.sample_start(logits, greedy)
        marks[step + 1].record()
    torch.cuda.synchronize()
    seconds = marks[0].elapsed_time(marks[-1]) / 1e3
    per_step = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
    launches = ops.launch_count() - launches_before
    clocks = sampler.stop() if sampler else None
    # which form of each product the step ran: the launchers' names of the last capture this batch size replayed
    kernels = {}
    if graphs is not None and batch <= graphs.max_batch:
        key = (graphs.rung(batch), graphs.launch_class(graphs.rung(batch), max(engine.length(s) for s in slots)))
        for name in getattr(graphs.captured.get(key), "kernel_names", []):
            kernels[name] = kernels.get(name, 0) + 1
    for s in slots:
        engine.release_slot(s)
    return {"seconds": seconds, "kernels": kernels, "tokens_per_second": batch * steps / seconds, "ms_per_step": 1e3 * seconds / steps,
            "ms_per_step_p50": percentile(per_step, 0.50), "ms_per_step_p95": percentile(per_step, 0.95),
            "kv_tokens_per_step": kv_total / steps, "launches": launches, "clocks": clocks}


def percentile(ordered, fraction):
    """Nearest-rank percentile of an ascending list (integrallis/models, models-bench/.../BenchmarkStatistics.java:35-59)."""
    if not ordered:
        return None
    rank = max(1, -(-int(round(fraction * 1000)) * len(ordered) // 1000))
    return ordered[min(len(ordered), rank) - 1]


def e2e_decode(model, batch, steps, warmup, prompt=PROMPT_TOKENS):
    """The same through generate_batch: host ids in, host ids out; rate over the decode steps
    (tokens after each request's first, as integrallis/models' TrialMeasurement counts them)."""
    from models_b200 import SamplingOptions

    vocab = model.metadata.vocab_size
    prompts = random_prompts(batch, prompt, vocab, 2)
    stamps = []

    def on_token(index, token):
        if index == 0:
            stamps.append(time.perf_counter())

    first = model.generate_batch(prompts, SamplingOptions(temperature=0.0, max_tokens=warmup + 1))  # warm-up
    results = model.generate_batch(prompts, SamplingOptions(temperature=0.0, max_tokens=steps + 1), on_token=on_token)
    seconds = stamps[-1] - stamps[0]
    # what was generated, as a hash (integrallis/models prints one per run, models-bench/.../SessionBatchProfileCli.java:287-293),
    # and whether the warm-up run -- the same prompts, fewer tokens -- produced the same ids as far as it went
    digest = hashlib.sha256()
    for result in results:
        digest.update(",".join(str(t) for t in result.tokens).encode() + b";")
    repeated = all(a.tokens == b.tokens[: len(a.tokens)] for a, b in zip(first, results))
    graphs = model.engine.decode_graphs
    h2d = 0  # the step's indices; the ids themselves stay on the device
    if graphs and graphs.captured:
        layout = next(c for (size, _), c in graphs.captured.items() if size == graphs.rung(batch)).layout
        h2d = 4 * (layout.total - layout.tokens)
    return {"tokens_per_second": batch * (len(stamps) - 1) / seconds, "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": 4 * batch, "tokens_hash": digest.hexdigest()[:16], "repeated": repeated}


def device_prefill(model, tokens, repeats=5):
    import torch

    from models_b200.engine import StepEntry

    engine = model.engine
    prompt = random_prompts(1, tokens, engine.spec.vocab_size, 3)[0]
    times = []
    warm = 4  # (a class of prompt steps is captured when it comes up for the third time: that run is part of the warm-up)
    for _ in range(repeats + warm):
        slot = engine.open_slot()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step([StepEntry(slot, prompt, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
        engine.release_slot(slot)
    return statistics.median(times[warm:])


# ------------------------------------------------------------------------------------------------
# --design kabanex: the Kabanex decoder beside a Llama of equal size (same width, layers, heads, key/value
# heads, window, vocabulary, and a feed-forward width that makes the layers' parameters equal), random
# weights, prefill and decode through the engine, and the design's own kernels alone beside their Llama
# counterparts.  The default run of this file does not come here.

DESIGN_SIZES = {
    # width, layers, heads, kv_heads, key size, value size, recurrent width, ff, window, kept first positions
    "s": dict(width=1024, layers=8, heads=8, kv_heads=2, dim=64, vdim=128, recurrent=1024, ff=2048, window=512, keep_first=4),
    "m": dict(width=2048, layers=16, heads=16, kv_heads=4, dim=64, vdim=128, recurrent=2048, ff=4096, window=1024, keep_first=4),
}
DESIGN_VOCAB = 32768


def kabanex_config(z):
    layer = {"type": "parallel",
             "mixer": {"left": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"],
                                "scale": z["dim"] ** -0.5, "rot": {"dims": z["dim"] // 2, "base": 500000.0},
                                "mask": {"size": z["window"], "keep_first": z["keep_first"]}},
                       "right": {"width": z["recurrent"]}, "left_scale": 1.0, "right_scale": 1.0},
             "mlp": {"kind": "dense", "ff": z["ff"]}}
    return {"architecture": "Kabanex", "vocab": DESIGN_VOCAB, "width": z["width"], "norm": {"eps": 1e-6},
            "layers": [layer] * z["layers"]}


def kabanex_layer_params(z):
    w, h, g = z["width"], z["heads"], z["kv_heads"]
    first = h * z["dim"] + g * z["dim"] + g * z["vdim"] + h + 3 * z["recurrent"] + z["ff"]
    return w * first + w * (h * z["vdim"] + z["recurrent"] + z["ff"])


def llama_like(z):
    """A Llama with the same width, layers, heads, key/value heads and window, heads of 128 (queries and values as
    wide as the design's values), and the feed-forward width that makes a layer's parameters equal (a multiple of 256)."""
    w, h, g, hd = z["width"], z["heads"], z["kv_heads"], 128
    attention = w * (h * hd + 2 * g * hd) + h * hd * w
    inter = max(256, round((kabanex_layer_params(z) - attention) / (3 * w) / 256) * 256)
    return dict(LLAMA_3_2_1B, num_hidden_layers=z["layers"], hidden_size=w, num_attention_heads=h, num_key_value_heads=g,
                head_dim=hd, intermediate_size=inter, vocab_size=DESIGN_VOCAB, sliding_window=z["window"], rope_scaling=None,
                tie_word_embeddings=False, max_position_embeddings=8192)


def time_kernel(call, repeats=7):
    """Median device time of `call()` in microseconds, L2 flushed before every run.  The call is replayed from a CUDA
    graph, as the engine replays its steps: launched from Python, a kernel of a few microseconds would be timed by the
    host's way to the launch (10 to 30 us per call), not by the device."""
    import torch

    flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device="cuda")  # 256 MB > 126 MB of L2
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        call()
    graph.replay()
    times = []
    for _ in range(repeats):
        flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) * 1e3)
    return statistics.median(times)


def design_kernels(z, peak, prompt=2048, batch=8, context=1536):
    """The design's kernels alone beside the like Llama kernels at equal sizes: attention over a prompt and in a
    decode step, the recurrence, the norm; each with its fraction of the measured peak that bounds it."""
    import torch

    from models_b200.kernels import ops

    dev, bf = "cuda", torch.bfloat16
    H, G, D, DV, R, W, window, keep = (z[k] for k in ("heads", "kv_heads", "dim", "vdim", "recurrent", "width", "window", "keep_first"))
    page = 64
    out = {}

    def paged(sequences, length, key, value):
        pages = sequences * (-(-length // page))
        k_pool = torch.randn((pages + 1, G, page, key), device=dev).to(bf)
        v_pool = torch.randn((pages + 1, G, page, value), device=dev).to(bf)
        table = (torch.arange(pages, dtype=torch.int32, device=dev) + 1).reshape(sequences, -1).contiguous()
        return k_pool, v_pool, table

    def seen(length, q_len):  # (query, key) pairs a step of q_len tokens ending at `length` looks at
        return sum(min(p + 1, window) + min(keep, max(0, p + 1 - window)) for p in range(length - q_len, length))

    # a prompt of `prompt` tokens, one sequence
    cu, kv = torch.tensor([0, prompt], dtype=torch.int32, device=dev), torch.tensor([prompt], dtype=torch.int32, device=dev)
    pairs = seen(prompt, prompt)
    k_pool, v_pool, table = paged(1, prompt, D, DV)
    q, o = torch.randn((prompt, H * D), device=dev).to(bf), torch.empty((prompt, H * DV), dtype=bf, device=dev)
    talk, gate = torch.randn((H, H), device=dev), torch.randn((prompt, H), device=dev).to(bf)
    us = time_kernel(lambda: ops.talking_attention(q, o, k_pool, v_pool, table, cu, kv, prompt, H, G, D, DV, window, keep, D ** -0.5, talk, gate))
    flops = pairs * H * (2 * D + 2 * DV + 2 * H)  # scores once, values once, the mixing; what the mechanism asks for
    out["prompt_attention_kabanex"] = {"us": us, "tflops": flops / us / 1e6, "frac_of_bf16_peak": flops / us / 1e6 / peak["bf16_tflops"]}
    hd = 128
    k2, v2, _ = paged(1, prompt, hd, hd)
    q2, o2 = torch.randn((prompt, H * hd), device=dev).to(bf), torch.empty((prompt, H * hd), dtype=bf, device=dev)
    us = time_kernel(lambda: ops.prefill_attention(q2, o2, k2, v2, table, cu, kv, prompt, H, G, hd, window, hd ** -0.5))
    flops = pairs * H * 4 * hd
    out["prompt_attention_llama"] = {"us": us, "tflops": flops / us / 1e6, "frac_of_bf16_peak": flops / us / 1e6 / peak["bf16_tflops"]}

    # a decode step of `batch` sequences that hold `context` positions
    cu = torch.arange(batch + 1, dtype=torch.int32, device=dev)
    kv = torch.full((batch,), context, dtype=torch.int32, device=dev)
    pairs = batch * seen(context, 1)
    k_pool, v_pool, table = paged(batch, context, D, DV)
    q, o = torch.randn((batch, H * D), device=dev).to(bf), torch.empty((batch, H * DV), dtype=bf, device=dev)
    gate = torch.randn((batch, H), device=dev).to(bf)
    us = time_kernel(lambda: ops.talking_attention(q, o, k_pool, v_pool, table, cu, kv, 1, H, G, D, DV, window, keep, D ** -0.5, talk, gate))
    moved = pairs * G * (D + DV) * 2
    out["decode_attention_kabanex"] = {"us": us, "gbs": moved / us / 1e3, "frac_of_hbm_peak": moved / us / 1e3 / peak["hbm_gbs"]}
    k2, v2, _ = paged(batch, context, hd, hd)
    q2, o2 = torch.randn((batch, H * hd), device=dev).to(bf), torch.empty((batch, H * hd), dtype=bf, device=dev)
    splits = ops.decode_splits(batch, H, G, hd, context, window, ops.multiprocessors(torch.device(dev)))
    us = time_kernel(lambda: ops.decode_attention(q2, o2, k2, v2, table, cu, kv, H, G, hd, window, hd ** -0.5, splits))
    moved = pairs * G * 2 * hd * 2
    out["decode_attention_llama"] = {"us": us, "gbs": moved / us / 1e3, "frac_of_hbm_peak": moved / us / 1e3 / peak["hbm_gbs"]}

    # the recurrence over a prompt and in a decode step; the layer norm beside the RMS norm
    state = torch.zeros((batch + 1, R), dtype=torch.float32, device=dev)
    zb, xb = torch.zeros(R, device=dev), torch.zeros(R, device=dev)
    for name, rows, cu_q, longest in (("prompt", prompt, [0, prompt], prompt), ("decode", batch, list(range(batch + 1)), 1)):
        proj, y = torch.randn((rows, 3 * R), device=dev).to(bf), torch.empty((rows, R), dtype=bf, device=dev)
        cu_t = torch.tensor(cu_q, dtype=torch.int32, device=dev)
        slots = torch.arange(len(cu_q) - 1, dtype=torch.int32, device=dev)
        us = time_kernel(lambda: ops.mingru_scan(proj[:, :R], proj[:, R:2 * R], proj[:, 2 * R:], zb, xb, state, slots, cu_t, longest, y))
        moved = rows * R * 2 * 4 + (len(cu_q) - 1) * R * 8
        out[f"{name}_recurrence"] = {"us": us, "gbs": moved / us / 1e3, "frac_of_hbm_peak": moved / us / 1e3 / peak["hbm_gbs"]}
    x = torch.randn((prompt, W), device=dev)
    gain, bias = torch.ones(W, device=dev), torch.zeros(W, device=dev)
    moved = prompt * W * 6
    us = time_kernel(lambda: ops.layernorm(x, gain, bias, 1e-6, bf))
    out["prompt_layernorm"] = {"us": us, "gbs": moved / us / 1e3, "frac_of_hbm_peak": moved / us / 1e3 / peak["hbm_gbs"]}
    us = time_kernel(lambda: ops.add_rmsnorm(x, None, gain, 1e-6, bf))
    out["prompt_rmsnorm_llama"] = {"us": us, "gbs": moved / us / 1e3, "frac_of_hbm_peak": moved / us / 1e3 / peak["hbm_gbs"]}
    return out


# --design lovurax: the Lovurax decoder (sigmoid attention, retention and latent attention layers in turn, gated
# residuals, an xIELU feed-forward) beside a Llama of equal size, the same way.

LOVURAX_SIZES = {
    # width, layers (attention, retention, attention, latent attention in turn), heads, key/value heads of the attention,
    # key size, value size, rank of the latent rows, ff
    "s": dict(width=1024, layers=8, heads=8, kv_heads=2, dim=64, vdim=128, rank=256, ff=2048),
    "m": dict(width=2048, layers=16, heads=16, kv_heads=4, dim=64, vdim=128, rank=256, ff=4096),
}
LOVURAX_ORDER = ("attention", "retention", "attention", "latent_attention")


def lovurax_config(z):
    H, D, DV = z["heads"], z["dim"], z["vdim"]
    mixers = {
        "attention": {"heads": H, "kv_heads": z["kv_heads"], "dim": D, "vdim": DV, "scale": D ** -0.5, "q_temp": {"coef": 0.4, "every": 128}},
        "retention": {"heads": H, "dim": D, "vdim": DV, "decay": [1.0 - 2.0 ** (-5 - 3 * h / max(1, H - 1)) for h in range(H)],
                      "rot": {"dims": D // 2, "base": 500000.0}},
        "latent_attention": {"heads": H, "dim": D, "vdim": DV, "kv_rank": z["rank"], "scale": D ** -0.5},
    }
    layers = [{"type": LOVURAX_ORDER[i % 4], "mixer": mixers[LOVURAX_ORDER[i % 4]], "mlp": {"kind": "dense", "ff": z["ff"]}}
              for i in range(z["layers"])]
    return {"architecture": "Lovurax", "vocab": DESIGN_VOCAB, "width": z["width"], "norm": {"eps": 1e-6}, "logit_scale": 1.0, "layers": layers}


def lovurax_layer_params(z):
    """Matrix parameters of a layer, averaged over the four layers of a turn."""
    w, h, g, d, dv, r = (z[k] for k in ("width", "heads", "kv_heads", "dim", "vdim", "rank"))
    mixer = {"attention": w * (h * d + g * d + g * dv + h * dv) + h * dv * w,
             "retention": w * (2 * h * d + 2 * h * dv) + h * dv * w,
             "latent_attention": w * (h * d + r + h) + r * (h * d + h * dv) + h * dv * w}
    return sum(mixer[kind] for kind in LOVURAX_ORDER) // 4 + 2 * w * w + 2 * w * z["ff"]


def llama_of_equal_size(z, layer_params):
    """A Llama with the same width, layers, heads and key/value heads, heads of 128 (queries and values as wide as the
    design's values), and the feed-forward width that makes a layer's parameters equal (a multiple of 256)."""
    w, h, g, hd = z["width"], z["heads"], z["kv_heads"], 128
    attention = w * (h * hd + 2 * g * hd) + h * hd * w
    inter = max(256, round((layer_params - attention) / (3 * w) / 256) * 256)
    return dict(LLAMA_3_2_1B, num_hidden_layers=z["layers"], hidden_size=w, num_attention_heads=h, num_key_value_heads=g,
                head_dim=hd, intermediate_size=inter, vocab_size=DESIGN_VOCAB, rope_scaling=None,
                tie_word_embeddings=False, max_position_embeddings=8192)


def lovurax_kernels(z, peak, prompt=2048, batch=8, context=1536):
    """The design's kernels alone beside the like kernels of the other models at equal sizes, each with its fraction
    of the measured peak that bounds it."""
    import torch

    from models_b200.kernels import ops

    dev, bf = "cuda", torch.bfloat16
    H, G, D, DV, R, W = (z[k] for k in ("heads", "kv_heads", "dim", "vdim", "rank", "width"))
    page = 64
    out = {}

    def paged(sequences, length, kv_heads, key, value):
        pages = sequences * (-(-length // page))
        k_pool = torch.randn((pages + 1, kv_heads, page, key), device=dev).to(bf)
        v_pool = torch.randn((pages + 1, kv_heads, page, value), device=dev).to(bf) if value else None
        table = (torch.arange(pages, dtype=torch.int32, device=dev) + 1).reshape(sequences, -1).contiguous()
        return k_pool, v_pool, table

    def rated(us, flops=None, moved=None):
        if flops is not None:
            return {"us": us, "tflops": flops / us / 1e6, "frac_of_bf16_peak": flops / us / 1e6 / peak["bf16_tflops"]}
        return {"us": us, "gbs": moved / us / 1e3, "frac_of_hbm_peak": moved / us / 1e3 / peak["hbm_gbs"]}

    hd = 128
    for name, rows, cu_q, lengths, q_len in (("prompt", prompt, [0, prompt], [prompt], prompt),
                                             ("decode", batch, list(range(batch + 1)), [context] * batch, 1)):
        sequences = len(lengths)
        cu = torch.tensor(cu_q, dtype=torch.int32, device=dev)
        kv = torch.tensor(lengths, dtype=torch.int32, device=dev)
        pairs = sum(sum(range(n - q_len + 1, n + 1)) for n in lengths)  # (query, key) pairs of a head
        # sigmoid attention: keys of D, values of DV, a gate per element
        k_pool, v_pool, table = paged(sequences, lengths[0], G, D, DV)
        q, o = torch.randn((rows, H * D), device=dev).to(bf), torch.empty((rows, H * DV), dtype=bf, device=dev)
        gate, bias = torch.randn((rows, H * DV), device=dev).to(bf), torch.zeros(H, device=dev)
        us = time_kernel(lambda: ops.gated_attention(q, o, k_pool, v_pool, table, cu, kv, q_len, H, G, D, DV, "sigmoid", D ** -0.5, 8.0,
                                                     bias, gate, "element"))
        out[f"{name}_sigmoid_attention"] = rated(us, flops=pairs * H * (2 * D + 2 * DV)) if q_len > 1 else \
            rated(us, moved=sum(lengths) * G * (D + DV) * 2)
        # latent attention: every head reads the rows of R as key and as value; the two small products per head around it
        c_pool, _, table = paged(sequences, lengths[0], 1, R, 0)
        ql, ol = torch.randn((rows, H * R), device=dev).to(bf) * 0.1, torch.empty((rows, H * R), dtype=bf, device=dev)
        us = time_kernel(lambda: ops.gated_attention(ql, ol, c_pool, None, table, cu, kv, q_len, H, 1, R, R, "softmax", D ** -0.5))
        out[f"{name}_latent_attention"] = rated(us, flops=pairs * H * 4 * R) if q_len > 1 else rated(us, moved=sum(lengths) * R * 2)
        into, back = torch.randn((H, R, D), device=dev).to(bf), torch.randn((H, DV, R), device=dev).to(bf)
        q_small, o_small = torch.randn((rows, H * D), device=dev).to(bf), torch.empty((rows, H * DV), dtype=bf, device=dev)
        us = time_kernel(lambda: (ops.head_linear(q_small, into, ql, H), ops.head_linear(ol, back, o_small, H)))
        out[f"{name}_latent_head_products"] = rated(us, flops=rows * H * 2 * R * (D + DV)) if q_len > 1 else \
            rated(us, moved=H * R * (D + DV) * 2)
        # the like Llama kernel: heads of 128
        k2, v2, table = paged(sequences, lengths[0], G, hd, hd)
        q2, o2 = torch.randn((rows, H * hd), device=dev).to(bf), torch.empty((rows, H * hd), dtype=bf, device=dev)
        if q_len > 1:
            us = time_kernel(lambda: ops.prefill_attention(q2, o2, k2, v2, table, cu, kv, q_len, H, G, hd, None, hd ** -0.5))
            out[f"{name}_attention_llama"] = rated(us, flops=pairs * H * 4 * hd)
        else:
            splits = ops.decode_splits(sequences, H, G, hd, lengths[0], None, ops.multiprocessors(torch.device(dev)))
            us = time_kernel(lambda: ops.decode_attention(q2, o2, k2, v2, table, cu, kv, H, G, hd, None, hd ** -0.5, splits))
            out[f"{name}_attention_llama"] = rated(us, moved=sum(lengths) * G * 2 * hd * 2)
        # retention beside the other recurrence of the package (minGRU over as many channels as the state has columns)
        state = torch.zeros((sequences + 1, H, D, DV), dtype=torch.float32, device=dev)
        proj = torch.randn((rows, 2 * H * D + 2 * H * DV), device=dev).to(bf)
        a, b, c = H * D, 2 * H * D, 2 * H * D + H * DV
        y = torch.empty((rows, H * DV), dtype=bf, device=dev)
        positions = torch.cat([torch.arange(n - q_len, n) for n in lengths]).to(torch.int32).to(dev)
        tables = torch.rand((max(lengths), D // 4), device=dev)
        decay = torch.full((H,), 0.99, device=dev)
        slots = torch.arange(sequences, dtype=torch.int32, device=dev)
        us = time_kernel(lambda: ops.retention_scan(proj[:, :a], proj[:, a:b], proj[:, b:c], proj[:, c:], positions, tables, tables, D // 2,
                                                    decay, D ** -0.5, 1e-6, state, slots, cu, H, D, DV, y, 1.0, q_len))
        # what must move: the projections and results once, the state in and out; the arithmetic: 2 x 2 D DV per token and head
        moved = rows * (2 * H * D + 3 * H * DV) * 2 + sequences * H * D * DV * 8
        out[f"{name}_retention"] = dict(rated(us, moved=moved), fp32_tflops=rows * H * 4 * D * DV / us / 1e6)
        width = H * DV
        gru_state = torch.zeros((sequences + 1, width), dtype=torch.float32, device=dev)
        gp, gy = torch.randn((rows, 3 * width), device=dev).to(bf), torch.empty((rows, width), dtype=bf, device=dev)
        zb = torch.zeros(width, device=dev)
        us = time_kernel(lambda: ops.mingru_scan(gp[:, :width], gp[:, width:2 * width], gp[:, 2 * width:], zb, zb, gru_state, slots, cu, q_len, gy))
        out[f"{name}_recurrence_kabanex"] = rated(us, moved=rows * width * 2 * 4 + sequences * width * 8)
    # element-wise: the gated residual add beside the plain one, the activation beside the gated one of Llama
    x, delta = torch.randn((prompt, W), device=dev), torch.randn((prompt, W), device=dev)
    gate, bias = torch.randn((prompt, W), device=dev).to(bf), torch.zeros(W, device=dev)
    out["prompt_gated_residual_add"] = rated(time_kernel(lambda: ops.gated_residual_add(x, gate, bias, delta)), moved=prompt * W * 14)
    out["prompt_residual_add_llama"] = rated(time_kernel(lambda: ops.residual_add(x, delta)), moved=prompt * W * 12)
    up, mid = torch.randn((prompt, z["ff"]), device=dev).to(bf), torch.empty((prompt, z["ff"]), dtype=bf, device=dev)
    out["prompt_xielu"] = rated(time_kernel(lambda: ops.xielu(up, mid, 0.7, 1.2)), moved=prompt * z["ff"] * 4)
    gate_up = torch.randn((prompt, 2 * z["ff"]), device=dev).to(bf)
    out["prompt_swiglu_llama"] = rated(time_kernel(lambda: ops.swiglu(gate_up)), moved=prompt * z["ff"] * 6)
    return out


# --design kivezen: the Kivezen decoder (capped attention with a sink and rotated values, lightning layers, routed
# experts, several residual streams) beside a Lovurax of equal size: the model of this package whose layers are nearest
# (attention over the same paged kernels, a retention walk); equal size counts the parameters a token uses.

KIVEZEN_SIZES = {
    # width, layers (KIVEZEN_ORDER in turn), heads, key/value heads, key size, value size, dense ff, experts, chosen per token,
    # an expert's ff, the shared expert's ff, residual streams; `rank` only sizes the Lovurax beside it
    "s": dict(width=1024, layers=8, heads=8, kv_heads=2, dim=64, vdim=128, ff=2048, experts=16, top=2, expert_ff=512, shared_ff=512,
              streams=2, rank=256),
    "m": dict(width=2048, layers=16, heads=16, kv_heads=4, dim=64, vdim=128, ff=4096, experts=32, top=4, expert_ff=512, shared_ff=1024,
              streams=4, rank=256),
}
KIVEZEN_ORDER = (("lightning", "dense"), ("attention", "moe"), ("attention", "dense"), ("lightning", "moe"))


def kivezen_config(z):
    H, D, DV = z["heads"], z["dim"], z["vdim"]
    mixers = {
        "attention": {"heads": H, "kv_heads": z["kv_heads"], "dim": D, "vdim": DV, "scale": D ** -0.5, "softcap": 50.0,
                      "rot": {"dims": D // 2, "base": 500000.0,
                              "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}},
        "lightning": {"heads": H, "dim": D, "vdim": DV, "decay": [1.0 - 2.0 ** (-5 - 3 * h / max(1, H - 1)) for h in range(H)]},
    }
    mlps = {"dense": {"kind": "dense", "ff": z["ff"]},
            "moe": {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": z["expert_ff"], "limit": 7.0},
                    "shared": {"ff": z["shared_ff"], "limit": 7.0}}}
    layers = []
    for i in range(z["layers"]):
        mixer, mlp = KIVEZEN_ORDER[i % 4]
        layers.append({"type": mixer, "mixer": mixers[mixer], "mlp": mlps[mlp]})
    return {"architecture": "Kivezen", "vocab": DESIGN_VOCAB, "width": z["width"], "norm": {"eps": 1e-6}, "streams": z["streams"],
            "logit_softcap": 30.0, "layers": layers}


def kivezen_layer_params(z):
    """Matrix parameters a token uses in a layer (of the experts only the chosen ones and the shared one), averaged over
    the four layers of a turn."""
    w, h, g, d, dv = (z[k] for k in ("width", "heads", "kv_heads", "dim", "vdim"))
    mixer = {"attention": w * (h * d + g * d + g * dv) + h * dv * w, "lightning": w * (2 * h * d + 2 * h * dv) + h * dv * w}
    mlp = {"dense": 2 * w * z["ff"], "moe": z["top"] * 3 * w * z["expert_ff"] + 3 * w * z["shared_ff"] + w * (z["experts"] + 1)}
    return sum(mixer[a] + mlp[b] for a, b in KIVEZEN_ORDER) // 4


def lovurax_of_equal_size(z):
    """A Lovurax of the same width, layers, heads and head sizes whose feed-forward width (a multiple of 256) makes a
    layer's parameters equal to those a Kivezen token uses."""
    w = z["width"]
    ff = max(256, round((kivezen_layer_params(z) - lovurax_layer_params(dict(z, ff=0))) / (2 * w) / 256) * 256)
    return lovurax_config(dict(z, ff=ff))


def kivezen_kernels(z, peak, prompt=2048, batch=8, context=1536):
    """The design's kernels alone beside the like kernels of the other models at equal sizes, each with its fraction of
    the measured peak that bounds it."""
    import torch

    from models_b200.kernels import ops
    from models_b200.parts.linear import linear

    dev, bf = "cuda", torch.bfloat16
    H, G, D, DV, W = (z[k] for k in ("heads", "kv_heads", "dim", "vdim", "width"))
    E, top, F, S = z["experts"], z["top"], z["expert_ff"], z["streams"]
    page = 64
    out = {}

    def paged(sequences, length, key, value):
        pages = sequences * (-(-length // page))
        k_pool = torch.randn((pages + 1, G, page, key), device=dev).to(bf)
        v_pool = torch.randn((pages + 1, G, page, value), device=dev).to(bf)
        table = (torch.arange(pages, dtype=torch.int32, device=dev) + 1).reshape(sequences, -1).contiguous()
        return k_pool, v_pool, table

    def rated(us, flops=None, moved=None):
        if flops is not None:
            return {"us": us, "tflops": flops / us / 1e6, "frac_of_bf16_peak": flops / us / 1e6 / peak["bf16_tflops"]}
        return {"us": us, "gbs": moved / us / 1e3, "frac_of_hbm_peak": moved / us / 1e3 / peak["hbm_gbs"]}

    longest = max(prompt, context)
    angle = torch.arange(longest, dtype=torch.float32, device=dev)[:, None]
    cos, sin = (f(angle * torch.rand((1, D // 4), device=dev)).contiguous() for f in (torch.cos, torch.sin))  # D / 2 coordinates turn
    vcos, vsin = (f(angle * torch.rand((1, DV // 2), device=dev)).contiguous() for f in (torch.cos, torch.sin))
    temperature = torch.rand(H, device=dev) + 0.5
    for name, rows, cu_q, lengths, q_len in (("prompt", prompt, [0, prompt], [prompt], prompt),
                                             ("decode", batch, list(range(batch + 1)), [context] * batch, 1)):
        sequences = len(lengths)
        cu = torch.tensor(cu_q, dtype=torch.int32, device=dev)
        kv = torch.tensor(lengths, dtype=torch.int32, device=dev)
        pairs = sum(sum(range(n - q_len + 1, n + 1)) for n in lengths)  # (query, key) pairs of a head
        positions = torch.cat([torch.arange(n - q_len, n) for n in lengths]).to(torch.int32).to(dev)
        # capped attention (a temperature per head, the cap, the sink, the turn back) beside the sigmoid attention of Lovurax
        k_pool, v_pool, table = paged(sequences, lengths[0], D, DV)
        q, o = torch.randn((rows, H * D), device=dev).to(bf), torch.empty((rows, H * DV), dtype=bf, device=dev)
        us = time_kernel(lambda: ops.gated_attention(q, o, k_pool, v_pool, table, cu, kv, q_len, H, G, D, DV, "softmax", D ** -0.5,
                                                     head_scale=temperature, softcap=50.0, sink=True, turn_cos=vcos, turn_sin=vsin))
        out[f"{name}_capped_attention"] = rated(us, flops=pairs * H * (2 * D + 2 * DV)) if q_len > 1 else \
            rated(us, moved=sum(lengths) * G * (D + DV) * 2)
        gate, bias = torch.randn((rows, H * DV), device=dev).to(bf), torch.zeros(H, device=dev)
        us = time_kernel(lambda: ops.gated_attention(q, o, k_pool, v_pool, table, cu, kv, q_len, H, G, D, DV, "sigmoid", D ** -0.5, 8.0,
                                                     bias, gate, "element"))
        out[f"{name}_sigmoid_attention_lovurax"] = rated(us, flops=pairs * H * (2 * D + 2 * DV)) if q_len > 1 else \
            rated(us, moved=sum(lengths) * G * (D + DV) * 2)
        # what stands before it: rotation, unit norm, rotated values, the pools; beside Lovurax's norm and store
        qkv = torch.randn((rows, (H + G) * D + G * DV), device=dev).to(bf)
        a, b = H * D, (H + G) * D
        mapping = (torch.arange(rows, dtype=torch.int32, device=dev) + page)
        moved = rows * (2 * H * D + 2 * G * D + 2 * G * DV) * 2
        us = time_kernel(lambda: ops.rotate_norm_store(qkv[:, :a], qkv[:, a:b], qkv[:, b:], positions, cos, sin, D // 2, True, True, 1e-6,
                                                       vcos, vsin, DV, k_pool, v_pool, mapping, H, G, D, DV))
        out[f"{name}_rotate_norm_store"] = rated(us, moved=moved)
        us = time_kernel(lambda: ops.norm_store(qkv[:, :a], qkv[:, a:b], qkv[:, b:], positions, None, None, 1e-6, 0.4, 128, k_pool, v_pool,
                                                mapping, H, G, D, DV))
        out[f"{name}_norm_store_lovurax"] = rated(us, moved=moved)
        # lightning (silu on the way in, no rotation, floats out, one norm over all heads and a sigmoid gate in a second
        # kernel) beside the retention of Lovurax (rotation, a norm per head and a silu gate in the walk)
        state = torch.zeros((sequences + 1, H, D, DV), dtype=torch.float32, device=dev)
        proj = torch.randn((rows, 2 * H * D + 2 * H * DV), device=dev).to(bf)
        a, b, c = H * D, 2 * H * D, 2 * H * D + H * DV
        y = torch.empty((rows, H * DV), dtype=bf, device=dev)
        raw = torch.empty((rows, H * DV), dtype=torch.float32, device=dev)
        decay = torch.full((H,), 0.99, device=dev)
        gain = torch.ones(H * DV, device=dev)
        slots = torch.arange(sequences, dtype=torch.int32, device=dev)
        moved = rows * (2 * H * D + 3 * H * DV) * 2 + sequences * H * D * DV * 8
        us = time_kernel(lambda: (ops.retention_scan(proj[:, :a], proj[:, a:b], proj[:, b:c], None, positions, None, None, 0, decay, 1.0, 1e-6,
                                                     state, slots, cu, H, D, DV, None, 1.0, q_len, input_activation="silu", raw_out=raw),
                                  ops.group_norm_gate(raw, gain, proj[:, c:], y, 1e-6, "sigmoid")))
        out[f"{name}_lightning"] = dict(rated(us, moved=moved + rows * H * DV * 8), fp32_tflops=rows * H * 4 * D * DV / us / 1e6)
        tables = torch.rand((longest, D // 4), device=dev)
        us = time_kernel(lambda: ops.retention_scan(proj[:, :a], proj[:, a:b], proj[:, b:c], proj[:, c:], positions, tables, tables, D // 2,
                                                    decay, D ** -0.5, 1e-6, state, slots, cu, H, D, DV, y, 1.0, q_len))
        out[f"{name}_retention_lovurax"] = dict(rated(us, moved=moved), fp32_tflops=rows * H * 4 * D * DV / us / 1e6)
        # routed experts (router, sorting, the two grouped products, the weighted sum) beside a dense gated feed-forward whose
        # width is what a token uses (top experts side by side), through the products the package gives a dense layer
        x = torch.randn((rows, W), device=dev).to(bf)
        router = (torch.randn((E, W), device=dev) * 0.02).to(bf)
        w_gate_up = (torch.randn((2, E, F, W), device=dev) * 0.02).to(bf)
        w_gate, w_up = w_gate_up[0], w_gate_up[1]
        w_down = (torch.randn((E, W, F), device=dev) * 0.02).to(bf)

        def routed():  # (as the model's feed-forward runs them)
            chosen, weights = ops.router_topk(x, router, top)
            if chosen.numel() <= ops.EXPERT_ROWS_ENTRIES:
                mid = ops.expert_rows_first(x, w_gate, w_up, chosen, 7.0, 1.702)
                return ops.expert_combine(ops.expert_rows_second(mid, w_down, chosen), weights)
            if chosen.numel() >= ops.GROUPED_ROWS_PER_EXPERT * E:
                plan = ops.route_pad(chosen, E)
                mid = ops.grouped_first_product(ops.gather_rows(x, plan), w_gate_up, plan, 7.0, 1.702)
                return ops.expert_combine(ops.grouped_second_product(mid, w_down, plan), weights, position=plan.position)
            plan = ops.route_sort(chosen, E)
            mid = ops.expert_first_product(x, w_gate, w_up, plan, 7.0, 1.702)
            return ops.expert_combine(ops.expert_second_product(mid, w_down, plan), weights)

        us = time_kernel(routed)
        flops = rows * top * 6 * W * F
        touched = min(E, rows * top)  # (about: experts whose matrices a small step reads)
        out[f"{name}_routed_experts"] = rated(us, flops=flops) if q_len > 1 else rated(us, moved=touched * 3 * W * F * 2)
        dense_in = (torch.randn((2 * top * F, W), device=dev) * 0.02).to(bf)
        dense_out = (torch.randn((W, top * F), device=dev) * 0.02).to(bf)
        dense_mid = torch.empty((rows, top * F), dtype=bf, device=dev)

        def dense():
            both = linear(x, dense_in, bf)
            ops.clamped_swish(both[:, :top * F], both[:, top * F:], dense_mid, 7.0, 1.702)
            return linear(dense_mid, dense_out, torch.float32)

        us = time_kernel(dense)
        out[f"{name}_dense_of_equal_use"] = rated(us, flops=flops) if q_len > 1 else rated(us, moved=top * 3 * W * F * 2)
        # the residual streams: reading (weighted sum and norm) and writing (mixing and addition) beside the one-stream kernels
        streams = torch.randn((rows, S * W), device=dev)
        delta = torch.randn((rows, W), device=dev)
        read, write, mix = torch.rand(S, device=dev), torch.rand(S, device=dev), torch.rand((S, S), device=dev)
        ones = torch.ones(W, device=dev)
        us = time_kernel(lambda: ops.hyper_read_norm(streams, read, ones, 1e-6, bf))
        out[f"{name}_streams_read_norm"] = rated(us, moved=rows * W * (4 * S + 2))
        us = time_kernel(lambda: ops.hyper_write(streams, delta, write, mix))
        out[f"{name}_streams_write"] = rated(us, moved=rows * W * (8 * S + 4))
        us = time_kernel(lambda: ops.hyper_write_read_norm(streams, delta, write, mix, read, ones, 1e-6, bf))  # as the blocks run them
        out[f"{name}_streams_write_and_read_norm"] = rated(us, moved=rows * W * (8 * S + 4 + 2))
        one = torch.randn((rows, W), device=dev)
        us = time_kernel(lambda: ops.add_rmsnorm(one, None, ones, 1e-6, bf))
        out[f"{name}_rmsnorm_llama"] = rated(us, moved=rows * W * 6)
        us = time_kernel(lambda: ops.residual_add(one, delta))
        out[f"{name}_residual_add_llama"] = rated(us, moved=rows * W * 12)
    return out


# --design rolevik: the Rolevik decoder (layers with the norm on the sublayers' results; an attention over chunks beside a gated
# delta rule; recurrent blocks around a gated linear recurrence; routed experts with a scored router, groups and identity
# experts) beside a Kivezen of equal size: the model of this package whose layers are nearest (attention through the same paged
# kernels, a recurrence with a matrix of state per head, routed experts); equal size counts the parameters a token uses.

ROLEVIK_SIZES = {
    # width, layers (ROLEVIK_ORDER in turn), the attention's heads, key/value heads, key size, value size and chunk, the delta
    # rule's heads and query/key heads (same key and value sizes), the recurrent block's width and blocks, dense ff, experts,
    # identity experts, chosen per token, groups (count, kept), an expert's ff, the shared expert's ff
    "s": dict(width=1024, layers=8, heads=8, kv_heads=2, dim=64, vdim=128, chunk=512, delta_heads=8, delta_kv_heads=4, recurrent=1024,
              blocks=4, ff=2048, experts=16, identity=4, top=2, groups=(4, 2), expert_ff=512, shared_ff=512),
    "m": dict(width=2048, layers=16, heads=16, kv_heads=4, dim=64, vdim=128, chunk=1024, delta_heads=16, delta_kv_heads=8, recurrent=2048,
              blocks=8, ff=4096, experts=32, identity=8, top=4, groups=(8, 4), expert_ff=512, shared_ff=1024),
}
ROLEVIK_ORDER = (("parallel", "dense"), ("rglru", "moe"), ("parallel", "moe"), ("rglru", "dense"))


def rolevik_config(z):
    D, DV = z["dim"], z["vdim"]
    mixers = {
        "parallel": {"left": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": D, "vdim": DV, "scale": D ** -0.5,
                              "mask": {"size": z["chunk"]}, "rot": {"dims": D // 2, "base": 500000.0}},
                     "right": {"heads": z["delta_heads"], "kv_heads": z["delta_kv_heads"], "dim": D, "vdim": DV, "conv": 4}},
        "rglru": {"width": z["recurrent"], "blocks": z["blocks"], "conv": 4},
    }
    mlps = {"dense": {"kind": "dense", "ff": z["ff"]},
            "moe": {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "shared": {"ff": z["shared_ff"]},
                    "router": {"experts": z["experts"], "identity": z["identity"], "top": z["top"], "scale": 2.0,
                               "groups": {"count": z["groups"][0], "keep": z["groups"][1]}}}}
    layers = []
    for i in range(z["layers"]):
        mixer, mlp = ROLEVIK_ORDER[i % 4]
        layers.append({"type": mixer, "mixer": mixers[mixer], "mlp": mlps[mlp]})
    return {"architecture": "Rolevik", "vocab": DESIGN_VOCAB, "width": z["width"], "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "logit_scale": 1.0, "layers": layers}


def rolevik_layer_params(z):
    """Matrix parameters a token uses in a layer (of the experts only the chosen ones and the shared one), averaged over the
    four layers of a turn."""
    w, h, g, d, dv, dh, dg, r = (z[k] for k in ("width", "heads", "kv_heads", "dim", "vdim", "delta_heads", "delta_kv_heads", "recurrent"))
    mixer = {"parallel": w * (h * d + g * d + g * dv) + h * dv * w + w * (2 * dg * d + 2 * dh * dv + 2 * dh) + dh * dv * w,
             "rglru": 3 * w * r + 2 * r * (r // z["blocks"])}
    mlp = {"dense": 3 * w * z["ff"], "moe": z["top"] * 3 * w * z["expert_ff"] + 3 * w * z["shared_ff"] + w * (z["experts"] + z["identity"])}
    return sum(mixer[a] + mlp[b] for a, b in ROLEVIK_ORDER) // 4


def kivezen_of_equal_size(z):
    """A Kivezen with one residual stream, of the same width, layers, heads, head sizes and experts, whose dense feed-forward
    width (a multiple of 256) makes a layer's parameters equal to those a Rolevik token uses."""
    zk = dict(z, streams=1, ff=0)
    ff = max(256, round((rolevik_layer_params(z) - kivezen_layer_params(zk)) / z["width"] / 256) * 256)  # (half the layers are dense: 2 w ff / 2)
    config = kivezen_config(dict(zk, ff=ff))
    del config["streams"]  # a plain residual sum
    return config


def rolevik_kernels(z, peak, prompt=2048, batch=8, context=1536):
    """The design's kernels alone beside the like kernels of the other models at equal sizes, each with its fraction of the
    measured peak that bounds it."""
    import torch

    from models_b200.kernels import ops

    dev, bf = "cuda", torch.bfloat16
    H, G, D, DV, W = (z[k] for k in ("heads", "kv_heads", "dim", "vdim", "width"))
    DH, DG, R, B = z["delta_heads"], z["delta_kv_heads"], z["recurrent"], z["blocks"]
    E, I, top, F = z["experts"], z["identity"], z["top"], z["expert_ff"]
    page, taps = 64, 4
    out = {}

    def paged(sequences, length, key, value):
        pages = sequences * (-(-length // page))
        k_pool = torch.randn((pages + 1, G, page, key), device=dev).to(bf)
        v_pool = torch.randn((pages + 1, G, page, value), device=dev).to(bf)
        table = (torch.arange(pages, dtype=torch.int32, device=dev) + 1).reshape(sequences, -1).contiguous()
        return k_pool, v_pool, table

    def rated(us, flops=None, moved=None):
        if flops is not None:
            return {"us": us, "tflops": flops / us / 1e6, "frac_of_bf16_peak": flops / us / 1e6 / peak["bf16_tflops"]}
        return {"us": us, "gbs": moved / us / 1e3, "frac_of_hbm_peak": moved / us / 1e3 / peak["hbm_gbs"]}

    longest = max(prompt, context)
    angle = torch.arange(longest, dtype=torch.float32, device=dev)[:, None]
    cos, sin = (f(angle * torch.rand((1, D // 4), device=dev)).contiguous() for f in (torch.cos, torch.sin))  # D / 2 coordinates turn
    vcos, vsin = (f(angle * torch.rand((1, DV // 2), device=dev)).contiguous() for f in (torch.cos, torch.sin))
    temperature = torch.rand(H, device=dev) + 0.5
    chunk = z["chunk"]
    for name, rows, cu_q, lengths, q_len in (("prompt", prompt, [0, prompt], [prompt], prompt),
                                             ("decode", batch, list(range(batch + 1)), [context] * batch, 1)):
        sequences = len(lengths)
        cu = torch.tensor(cu_q, dtype=torch.int32, device=dev)
        kv = torch.tensor(lengths, dtype=torch.int32, device=dev)
        slots = torch.arange(sequences, dtype=torch.int32, device=dev)
        # (query, key) pairs of a head: inside the query's chunk only; in all for the attention without chunks beside it
        seen = sum(p % chunk + 1 for n in lengths for p in range(n - q_len, n))
        pairs = sum(sum(range(n - q_len + 1, n + 1)) for n in lengths)
        positions = torch.cat([torch.arange(n - q_len, n) for n in lengths]).to(torch.int32).to(dev)
        k_pool, v_pool, table = paged(sequences, lengths[0], D, DV)
        q, o = torch.randn((rows, H * D), device=dev).to(bf), torch.empty((rows, H * DV), dtype=bf, device=dev)
        us = time_kernel(lambda: ops.gated_attention(q, o, k_pool, v_pool, table, cu, kv, q_len, H, G, D, DV, "softmax", D ** -0.5, block=chunk))
        out[f"{name}_chunked_attention"] = rated(us, flops=seen * H * (2 * D + 2 * DV)) if q_len > 1 else \
            rated(us, moved=sum(n - 1 - (n - 1) // chunk * chunk + 1 for n in lengths) * G * (D + DV) * 2)
        us = time_kernel(lambda: ops.gated_attention(q, o, k_pool, v_pool, table, cu, kv, q_len, H, G, D, DV, "softmax", D ** -0.5,
                                                     head_scale=temperature, softcap=50.0, sink=True, turn_cos=vcos, turn_sin=vsin))
        out[f"{name}_capped_attention_kivezen"] = rated(us, flops=pairs * H * (2 * D + 2 * DV)) if q_len > 1 else \
            rated(us, moved=sum(lengths) * G * (D + DV) * 2)
        # what stands before it: biases, one norm over each whole projection, rotation, the pools; beside Kivezen's kernel
        qkv = torch.randn((rows, (H + G) * D + G * DV), device=dev).to(bf)
        a, b = H * D, (H + G) * D
        mapping = (torch.arange(rows, dtype=torch.int32, device=dev) + page)
        moved = rows * (2 * H * D + 2 * G * D + 2 * G * DV) * 2
        bq, bk, bv, gq, gk = (torch.randn(n, device=dev) for n in (H * D, G * D, G * DV, H * D, G * D))
        us = time_kernel(lambda: ops.project_norm_rotate_store(qkv[:, :a], qkv[:, a:b], qkv[:, b:], bq, bk, bv, gq, gk, 1e-6, positions, cos, sin,
                                                               D // 2, False, k_pool, v_pool, mapping, H, G, D, DV))
        out[f"{name}_project_norm_rotate_store"] = rated(us, moved=moved)
        us = time_kernel(lambda: ops.rotate_norm_store(qkv[:, :a], qkv[:, a:b], qkv[:, b:], positions, cos, sin, D // 2, True, True, 1e-6,
                                                       vcos, vsin, DV, k_pool, v_pool, mapping, H, G, D, DV))
        out[f"{name}_rotate_norm_store_kivezen"] = rated(us, moved=moved)
        # the gated delta rule (convolution, its stored inputs, the walk with norm and gate) beside Kivezen's lightning layer
        C = 2 * DG * D + DH * DV
        floats = DH * D * DV
        state = torch.zeros((sequences + 1, floats + (taps - 1) * C), dtype=torch.float32, device=dev)
        proj = torch.randn((rows, C + 16 + DH * DV), device=dev).to(bf)
        conv_w = torch.randn((C, taps), device=dev)
        decay, dt_bias, gain = -torch.rand(DH, device=dev), torch.randn(DH, device=dev), torch.ones(DV, device=dev)
        y = torch.empty((rows, DH * DV), dtype=bf, device=dev)

        def delta():
            conv = ops.short_conv(proj[:, :C], conv_w, state, floats, slots, cu, q_len, activation="silu", store_tail=True)
            ops.gated_delta_scan(conv, 0, DG * D, 2 * DG * D, proj[:, C:C + DH], proj[:, C + 8:C + 8 + DH], proj[:, C + 16:], decay, dt_bias, gain,
                                 1e-6, 1e-6, state, 0, slots, cu, DH, DG, D, DV, y)

        us = time_kernel(delta)
        moved = rows * (C * 2 + C * 8 + 2 * DH * DV * 2) + sequences * floats * 8
        out[f"{name}_gated_delta_rule"] = dict(rated(us, moved=moved), fp32_tflops=rows * DH * 6 * D * DV / us / 1e6)
        us = time_kernel(lambda: ops.gated_delta_scan(ops.short_conv(proj[:, :C], conv_w, state, floats, slots, cu, q_len, activation="silu"), 0,
                                                      DG * D, 2 * DG * D, proj[:, C:C + DH], proj[:, C + 8:C + 8 + DH], proj[:, C + 16:], decay,
                                                      dt_bias, gain, 1e-6, 1e-6, state, 0, slots, cu, DH, DG, D, DV, y)) - \
            time_kernel(lambda: ops.short_conv(proj[:, :C], conv_w, state, floats, slots, cu, q_len, activation="silu"))
        out[f"{name}_gated_delta_rule_walk_alone"] = {"us": us, "fp32_tflops": rows * DH * 6 * D * DV / us / 1e6}
        lstate = torch.zeros((sequences + 1, DH, D, DV), dtype=torch.float32, device=dev)
        lproj = torch.randn((rows, 2 * DH * D + 2 * DH * DV), device=dev).to(bf)
        a, b, c = DH * D, 2 * DH * D, 2 * DH * D + DH * DV
        raw = torch.empty((rows, DH * DV), dtype=torch.float32, device=dev)
        ldecay, lgain = torch.full((DH,), 0.99, device=dev), torch.ones(DH * DV, device=dev)
        us = time_kernel(lambda: (ops.retention_scan(lproj[:, :a], lproj[:, a:b], lproj[:, b:c], None, positions, None, None, 0, ldecay, 1.0, 1e-6,
                                                     lstate, slots, cu, DH, D, DV, None, 1.0, q_len, input_activation="silu", raw_out=raw),
                                  ops.group_norm_gate(raw, lgain, lproj[:, c:], y, 1e-6, "sigmoid")))
        out[f"{name}_lightning_kivezen"] = dict(rated(us, moved=rows * (2 * DH * D + 3 * DH * DV) * 2 + rows * DH * DV * 8 + sequences * floats * 8),
                                                fp32_tflops=rows * DH * 4 * D * DV / us / 1e6)
        # the recurrent block (convolution, the gates' small products, the walk) beside Kabanex's minGRU walk of equal width
        rstate = torch.zeros((sequences + 1, R * taps), dtype=torch.float32, device=dev)
        rproj = torch.randn((rows, 3 * R), device=dev).to(bf)
        rconv, gates_w = torch.randn((R, taps), device=dev), torch.randn((B, 2 * (R // B), R // B), device=dev) * 0.05
        gates_twice = torch.cat([gates_w, gates_w], dim=2).to(bf).contiguous()
        vec = [torch.randn(R, device=dev) for _ in range(5)]
        rate = -8.0 * torch.rand(R, device=dev)
        ry = torch.empty((rows, R), dtype=bf, device=dev)

        def recurrent():
            sums = torch.empty((rows, 2 * R), dtype=torch.float32, device=dev)
            if rows > ops.WIDE_ROWS:  # (as the part runs them: a prompt's gate products on the tensor cores, u as two bfloat16 numbers)
                u, split = ops.short_conv(rproj[:, R:2 * R], rconv, rstate, R, slots, cu, q_len, in_bias=vec[0], out_bias=vec[1],
                                          store_tail=True, split_per=R // B)
                for blk in range(B):
                    at = blk * 2 * (R // B)
                    ops.gemm_tcgen05(split[:, at:at + 2 * (R // B)], gates_twice[blk], ops.EPI_F32, out=sums[:, at:at + 2 * (R // B)])
            else:
                u = ops.short_conv(rproj[:, R:2 * R], rconv, rstate, R, slots, cu, q_len, in_bias=vec[0], out_bias=vec[1], store_tail=True)
                ops.head_linear(u, gates_w, sums, B, tensor_cores=False)
            ops.rglru_scan(sums, R // B, u, rproj[:, :R], vec[2], vec[3], vec[4], rate, rstate, 0, slots, cu, q_len, ry)

        us = time_kernel(recurrent)
        out[f"{name}_recurrent_block"] = dict(rated(us, moved=rows * R * (2 + 4 + 4 + 8 + 8 + 4 + 2 + 2)), gate_products_tflops=rows * 4 * R * (R // B) / us / 1e6)
        mstate = torch.zeros((sequences + 1, R), dtype=torch.float32, device=dev)
        us = time_kernel(lambda: ops.mingru_scan(rproj[:, :R], rproj[:, R:2 * R], rproj[:, 2 * R:], vec[0], vec[1], mstate, slots, cu, q_len, ry))
        out[f"{name}_mingru_walk_kabanex"] = rated(us, moved=rows * R * 8)
        # routed experts: a scored router with a correction and groups, identity experts, the plain gated form; beside Kivezen's
        x = torch.randn((rows, W), device=dev).to(bf)
        router = (torch.randn((E + I, W), device=dev) * 0.02).to(bf)
        router_k = router[:E].contiguous()
        correction = torch.randn(E + I, device=dev) * 0.01
        w_gate_up = (torch.randn((2, E, F, W), device=dev) * 0.02).to(bf)
        w_gate, w_up = w_gate_up[0], w_gate_up[1]
        w_down = (torch.randn((E, W, F), device=dev) * 0.02).to(bf)
        inf = float("inf")

        def routed(scored):
            if scored:
                chosen, weights = ops.router_topk(x, router, top, scored=True, correction=correction, groups=z["groups"][0], keep=z["groups"][1],
                                                  weight_scale=2.0)
                limit, slope, offset, extra = inf, 1.0, 0.0, dict(chosen=chosen, experts=E, rows=x)
            else:
                chosen, weights = ops.router_topk(x, router_k, top)
                limit, slope, offset, extra = 7.0, 1.702, 1.0, {}
            if chosen.numel() <= ops.EXPERT_ROWS_ENTRIES:
                mid = ops.expert_rows_first(x, w_gate, w_up, chosen, limit, slope, offset)
                return ops.expert_combine(ops.expert_rows_second(mid, w_down, chosen), weights, **extra)
            if chosen.numel() >= ops.GROUPED_ROWS_PER_EXPERT * E:
                plan = ops.route_pad(chosen, E)
                mid = ops.grouped_first_product(ops.gather_rows(x, plan), w_gate_up, plan, limit, slope, offset)
                return ops.expert_combine(ops.grouped_second_product(mid, w_down, plan), weights, position=plan.position, **extra)
            plan = ops.route_sort(chosen, E)
            mid = ops.expert_first_product(x, w_gate, w_up, plan, limit, slope, up_offset=offset)
            return ops.expert_combine(ops.expert_second_product(mid, w_down, plan), weights, **extra)

        flops = rows * top * 6 * W * F  # (an upper bound for the design: identity experts' entries skip the products)
        touched = min(E, rows * top)
        for title, scored in (("routed_experts", True), ("routed_experts_kivezen", False)):
            us = time_kernel(lambda: routed(scored))
            out[f"{name}_{title}"] = rated(us, flops=flops) if q_len > 1 else rated(us, moved=touched * 3 * W * F * 2)
        # the norm on a sublayer's result, the scale, the addition and the copy for the next reader in one kernel; beside the
        # residual add and RMS norm of a pre-norm layer
        stream, res, res2 = (torch.randn((rows, W), device=dev) for _ in range(3))
        ones = torch.ones(W, device=dev)
        us = time_kernel(lambda: ops.outnorm_add(stream, res, ones, ones, 1e-6, copy_dtype=bf))
        out[f"{name}_result_norm_add"] = rated(us, moved=rows * W * (4 + 8 + 2))
        us = time_kernel(lambda: ops.outnorm_add(stream, res, ones, ones, 1e-6, b=res2, gain_a=ones, gain_b=ones, copy_dtype=bf))
        out[f"{name}_pair_result_norm_add"] = rated(us, moved=rows * W * (8 + 8 + 2))
        us = time_kernel(lambda: ops.add_rmsnorm(stream, res, ones, 1e-6, bf))
        out[f"{name}_add_rmsnorm_llama"] = rated(us, moved=rows * W * (4 + 8 + 2))
    return out


def design_run(args) -> int:
    import torch

    peak = peaks()
    batch, prompt, prefill_tokens, steps, warmup = 8, 512, 2048, args.steps or 64, max(args.warmup, 3)
    other, other_title = "llama", "LlamaForCausalLM of equal size"
    if args.design == "kabanex":
        title, all_sizes, make, params, beside, alone = "Kabanex", DESIGN_SIZES, kabanex_config, kabanex_layer_params, \
            (lambda z: llama_like(z)), design_kernels
    elif args.design == "kivezen":
        title, all_sizes, make, params, beside, alone = "Kivezen", KIVEZEN_SIZES, kivezen_config, kivezen_layer_params, \
            lovurax_of_equal_size, kivezen_kernels
        other, other_title = "lovurax", "Lovurax of equal size (the parameters a token uses)"
    elif args.design == "rolevik":
        title, all_sizes, make, params, beside, alone = "Rolevik", ROLEVIK_SIZES, rolevik_config, rolevik_layer_params, \
            kivezen_of_equal_size, rolevik_kernels
        other, other_title = "kivezen", "Kivezen of equal size (the parameters a token uses; one residual stream)"
    else:
        title, all_sizes, make, params, beside, alone = "Lovurax", LOVURAX_SIZES, lovurax_config, lovurax_layer_params, \
            (lambda z: llama_of_equal_size(z, lovurax_layer_params(z))), lovurax_kernels
    sizes = {}
    for name, z in all_sizes.items():
        if args.size and name != args.size:
            continue
        entry = {"sizes": z, "layer_params": params(z)}
        for arch, config in ((args.design, make(z)), (other, beside(z))):
            model = make_model(config, batch, prefill_tokens + 64)
            ms = device_prefill(model, prefill_tokens)
            run = device_decode(model, batch, steps, warmup, prompt=prompt)
            entry[arch] = {"prefill_tokens_per_s": prefill_tokens / (ms / 1e3), "prefill_ms": ms,
                           "decode_tokens_per_s": run["tokens_per_second"], "decode_ms_per_step": run["ms_per_step"],
                           "launches_per_step": run["launches"] / steps, "kernels": run["kernels"]}
            if arch == "llama":
                entry[arch]["intermediate_size"] = config["intermediate_size"]
            elif arch == other:
                entry[arch]["ff"] = config["layers"][0]["mlp"]["ff"]
            model.close()
            del model
            torch.cuda.empty_cache()
        entry["kernels_alone"] = alone(z, peak)
        sizes[name] = entry
    print(json.dumps({"design": title, "beside": other_title, "dtype": "bf16", "gpu": torch.cuda.get_device_name(0),
                      "data": "synthetic: seeded uniform-random token ids, random weights N(0, 0.02)",
                      "workload": {"prefill_tokens": prefill_tokens, "decode_batch": batch, "decode_prompt": prompt, "decode_steps": steps,
                                   "warmup": warmup, "vocab": DESIGN_VOCAB},
                      "peaks": peak, "sizes": sizes}))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None, help="decode steps timed (default: the workload's generated tokens)")
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--model", default="1b", choices=sorted(WORKLOADS),
                        help="1b: the default run; 3b, 8b: the other two workloads of the baseline file")
    parser.add_argument("--batch", type=int, default=None, help="sequences decoded together (default: the workload's)")
    parser.add_argument("--prompt", type=int, default=None,
                        help="prompt tokens per sequence (default: the workload's); the context grows to hold them")
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (both counts are reported)")
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 decode points and the prefill")
    parser.add_argument("--only-prefill", action="store_true",
                        help="run the workload's prefill alone and print its figures (for profiling)")
    parser.add_argument("--size", default=None, choices=["s", "m"], help="with --design: one of its two sizes alone")
    parser.add_argument("--design", default=None, choices=["kabanex", "lovurax", "kivezen", "rolevik"],
                        help="instead of the default run: this design beside a model of equal size (a Llama; for kivezen a Lovurax, for rolevik a Kivezen): "
                             "prefill, decode, its kernels alone")
    args = parser.parse_args()
    if args.design and args.impl == "ours":
        if args.gpus != 1:
            print(f"bench.py measures one GPU: --gpus {args.gpus} is not built")
            return 2
        return design_run(args)

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": (
            "integrallis/models is a Java 25 / Gradle library with a Rust crate and no Python package: pip cannot "
            "install it, and no JVM, Gradle or cargo is in this image")}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this library runs on a single GPU and --gpus {args.gpus} is not built")
        return 2
    warmup = max(args.warmup, 3)
    work = WORKLOADS[args.model]
    batch = args.batch or work["batch"]
    steps = args.steps or work["steps"]
    layers = args.layers or work["config"]["num_hidden_layers"]
    prompt, context, prefill_tokens = work["prompt"], work["context"], work["prefill"]
    if args.prompt:
        prompt, context = args.prompt, max(context, args.prompt + warmup + steps + 64)
    longest_prompt = prompt if isinstance(prompt, int) else prompt[1]
    if longest_prompt + warmup + steps + 1 > context:
        print(f"bench.py: {longest_prompt} prompt tokens + {warmup} + {steps} steps do not fit the context of {context}")
        return 2

    import torch

    config = dict(work["config"], num_hidden_layers=layers)
    peak = peaks()
    if args.only_prefill:
        model = make_model(config, 1, max(context, prefill_tokens + 64))
        ms = device_prefill(model, prefill_tokens, repeats=1)
        print(json.dumps({"prefill_ms": ms, "tokens": prefill_tokens}))
        return 0
    with_points = not args.no_points
    # the prefill fits the decode cache when it is no longer than a sequence's context; else it gets a model of its own
    prefill_fits = prefill_tokens + 64 <= context
    sequences = max([batch] + (list(work["points"]) if with_points else []))
    model = make_model(config, sequences, context)
    main_run = device_decode(model, batch, steps, warmup, sample_clocks=True, prompt=prompt)
    e2e = e2e_decode(model, batch, steps, warmup, prompt=prompt)
    bytes_per_step = decode_bytes(config, layers, main_run["kv_tokens_per_step"])
    achieved = bytes_per_step / (main_run["ms_per_step"] / 1e3) / 1e9
    weights_gb = decode_bytes(config, layers, 0) / 1e9

    line = {
        "metric": f"decode tok/s @ batch {batch} ({work['name'].split(' (')[0]}, bf16)",
        "value": main_run["tokens_per_second"],
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": main_run["ms_per_step"],
        "ms_per_step_p50": main_run["ms_per_step_p50"],
        "ms_per_step_p95": main_run["ms_per_step_p95"],
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: seeded uniform-random token ids, random weights N(0, 0.02)",
        "impl": "ours",
        "gpu": torch.cuda.get_device_name(0),
        "tokens_hash": e2e["tokens_hash"],
        "tokens_repeat_the_warmup_run": e2e["repeated"],
        "config": {
            "model": work["name"],
            "layers": layers,
            "layers_of_model": work["config"]["num_hidden_layers"],
            "hidden_size": config["hidden_size"],
            "heads": config["num_attention_heads"],
            "kv_heads": config["num_key_value_heads"],
            "head_dim": config["head_dim"],
            "intermediate_size": config["intermediate_size"],
            "vocab_size": config["vocab_size"],
            "tied_embeddings": bool(config["tie_word_embeddings"]),
            "global_batch": batch,
            "context_len": context,
            "prompt_len": prompt if isinstance(prompt, int) else f"{prompt[0]}..{prompt[1]} (unequal)",
            "seq_len": longest_prompt + warmup + steps,
            "parallelism": "single GPU",
            "sampling": "greedy",
            "cache": "paged, 64 positions per page, bf16",
            "l2": f"each step reads ~{weights_gb:.1f} GB of weights (> 126 MB L2); no flush needed",
            "peaks": peak["source"],
        },
        "e2e": {"value": e2e["tokens_per_second"], "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d_bytes_per_step"],
                "d2h_bytes_per_step": e2e["d2h_bytes_per_step"]},
        "gpu_launches": main_run["launches"],
        "kernels": main_run["kernels"],
        "clocks": main_run["clocks"],
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peak["hbm_gbs"], "bytes_per_step": bytes_per_step},
    }
    if with_points:
        points = {}
        for b in work["points"]:
            points[f"decode_b{b}"] = device_decode(model, b, min(steps, 64), warmup, prompt=prompt)["tokens_per_second"]
        if points:
            line["points"] = points
        if not prefill_fits:
            model.close()
            del model
            torch.cuda.empty_cache()
            model = make_model(config, 1, prefill_tokens + 64)
        ms = device_prefill(model, prefill_tokens)
        flops = prefill_flops(config, layers, prefill_tokens)
        line["prefill"] = {"value": prefill_tokens / (ms / 1e3), "tokens": prefill_tokens, "ms": ms,
                           "frac": flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12)}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
