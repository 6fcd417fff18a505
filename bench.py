#!/usr/bin/env python3
"""The benchmark the build driver runs: GPT-2 XL decode and prefill throughput on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on standard output. ``value`` is decoded tokens per second at batch 8 with
random bf16 weights of GPT-2 XL's sizes (``configs[2]`` of BASELINE.json): eight 512-token
prompts are prefilled, then W untimed and K timed decode steps run (context grows from
512 + W towards 1024), timed on the device with CUDA events around the K steps. A decode step
is the engine's own step: CUDA-graph replay of the whole forward plus token choice, fed from
pinned host memory, with the chosen ids read back. ``e2e`` is the same measured through the
Python entry point ``LLM.generate`` with host token ids in and out, as (time of T tokens -
time of 1 token) / (T - 1), the reference's method (``benchmarks/e2e/decode.py:1-10``).
``prefill`` is one 2,048-token step (two prompts of 1,024). ``roofline`` divides the bytes a
decode step must read (every weight once plus the live requests' keys and values) by its
time and by the measured copy bandwidth. ``points`` holds decode at batch 1 and 64.

``kernels`` holds, for the batch-8 decode step and for the prefill step, what each kernel
class costs inside the step (the step replayed as a CUDA graph with and without the class)
and its fraction of the roofline that bounds it. ``workloads`` holds the two serving
workloads of BASELINE.json's other configurations (see :func:`workload_run`);
``--workload small|large`` runs one of them alone and prints a line of its own.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

XL = {
    "architectures": ["GPT2LMHeadModel"], "n_layer": 48, "n_embd": 1600, "n_head": 25,
    "n_inner": 6400, "vocab_size": 50257, "n_positions": 1024, "layer_norm_epsilon": 1e-5,
    "activation_function": "gelu_new", "scale_attn_by_inverse_layer_idx": False,
    "tie_word_embeddings": True,
}
PROMPT = 512
METRIC = "decode tok/s at batch 8 (GPT-2 XL, bf16, context 1024)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            if "hbm_gbs" in data and "bf16_tflops" in data:
                return data, "measured"
        except (json.JSONDecodeError, OSError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class Clocks:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.process = None

    def start(self) -> None:
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.process = None

    def stop(self) -> dict:
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
        self.file.flush()
        self.file.seek(0)
        sm, peak, reasons = [], 0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.file.read().splitlines():
            fields = [field.strip() for field in line.split(",")]
            if len(fields) < 7:
                continue
            try:
                sm.append(int(float(fields[0])))
                peak = max(peak, int(float(fields[1])))
            except ValueError:
                continue
            for name, field in zip(names, fields[3:7]):
                if field.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": peak or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def layer_weight_bytes(cfg: dict, layers: int) -> int:
    d, f, v = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"]
    per_layer = (3 * d * d + d * d + 2 * d * f) * 2 + (3 * d + d + f + d + 4 * d) * 4
    return layers * per_layer + v * d * 2 + 2 * d * 4  # + tied head (wte) and ln_f


def kv_bytes_per_token(cfg: dict, layers: int) -> int:
    return layers * 2 * cfg["n_embd"] * 2


def prefill_flops(cfg: dict, layers: int, prompts: int, length: int) -> float:
    d, f, v = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"]
    tokens = prompts * length
    gemm = 2.0 * tokens * (3 * d * d + d * d + 2 * d * f) * layers
    attention = layers * prompts * 4.0 * d * (length * (length + 1) / 2)
    return gemm + attention + 2.0 * prompts * d * v


def build(cfg: dict, batch: int, tokens_per_step: int, seed: int = 0):
    import torch

    from ayaka_b200 import LLM, EngineConfig
    from ayaka_b200.weights.random_init import random_state

    state = random_state(cfg, seed, None, "bfloat16")
    with tempfile.TemporaryDirectory() as folder:
        (Path(folder) / "config.json").write_text(json.dumps(cfg))
        config = EngineConfig(
            model=folder, dtype="bfloat16", device="cuda:0", block_size=16,
            kv_reserve_tokens=batch * cfg["n_positions"], max_running=batch,
            max_tokens_per_step=tokens_per_step, cuda_graph=True)
        llm = LLM.from_config(config, tensors=state)
    del state
    torch.cuda.synchronize()
    return llm


def random_prompts(cfg: dict, count: int, length: int, seed: int) -> list[tuple[int, ...]]:
    import torch

    g = torch.Generator().manual_seed(seed)
    return [tuple(torch.randint(0, cfg["vocab_size"], (length,), generator=g).tolist())
            for _ in range(count)]


def decode_run(llm, cfg: dict, batch: int, warmup: int, steps: int, seed: int) -> dict:
    """Prefill ``batch`` prompts, then time ``steps`` decode steps after ``warmup`` untimed
    ones; returns device milliseconds per step and the contexts seen."""
    import torch

    from ayaka_b200 import SamplingParams
    from ayaka_b200.kernels import ops

    scheduler = llm.scheduler
    params = SamplingParams(temperature=0.0, max_tokens=None, ignore_eos=True)
    for index, prompt in enumerate(random_prompts(cfg, batch, PROMPT, seed)):
        scheduler.add_request(f"bench-{seed}-{index}", prompt, params)
    while any(request.prefilling for request in scheduler.running.values()) or scheduler.waiting:
        llm._advance()
    for _ in range(warmup):
        llm._advance()
    torch.cuda.synchronize()
    # with the next step launched ahead, the device is one step further than the host
    ahead = 1 if llm.graphs and llm.config.decode_ahead else 0
    first_context = PROMPT + 1 + warmup + ahead
    launches_before = ops.launch_count()
    replays_before = llm.graphs.replays if llm.graphs else 0
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall = time.perf_counter()
    start.record()
    for _ in range(steps):
        llm._advance()
    stop.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall
    ms = start.elapsed_time(stop) / steps
    replays = (llm.graphs.replays if llm.graphs else 0) - replays_before
    per_graph = 0
    if llm.graphs:
        bucket = llm.graphs.bucket_for(batch)
        per_graph = bucket.kernels
    launches = (ops.launch_count() - launches_before) + replays * per_graph
    for request_id in list(scheduler.running):
        scheduler.abort(request_id)
    scheduler.take_events()
    llm.core.manager.check_integrity()
    mean_context = first_context + (steps - 1) / 2
    return {"ms": ms, "wall_ms": wall * 1000 / steps, "mean_context": mean_context,
            "launches": launches, "replays": replays}


def prefill_run(llm, cfg: dict, warmup: int, repeats: int) -> dict:
    import torch

    from ayaka_b200.engine.runner import StepEntry

    length = cfg["n_positions"]
    times = []
    for index in range(warmup + repeats):
        prompts = random_prompts(cfg, 2, length, 900 + index)
        entries = [StepEntry(f"prefill-{index}-{i}", prompt, (length - 1,))
                   for i, prompt in enumerate(prompts)]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        llm.step(entries)
        stop.record()
        torch.cuda.synchronize()
        if index >= warmup:
            times.append(start.elapsed_time(stop))
        for entry in entries:
            llm.release(entry.request_id)
    times.sort()
    return {"ms": times[len(times) // 2], "tokens": 2 * length}


def e2e_run(llm, cfg: dict, batch: int, tokens: int) -> dict:
    """Decode tokens per second through ``LLM.generate``: host ids in, host ids out."""
    from ayaka_b200 import SamplingParams

    prompts = random_prompts(cfg, batch, PROMPT, 4242)

    def timed(max_tokens: int) -> float:
        begin = time.perf_counter()
        outputs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=max_tokens,
                                                       ignore_eos=True))
        elapsed = time.perf_counter() - begin
        assert all(len(o.outputs[0].token_ids) == max_tokens for o in outputs)
        return elapsed

    timed(4)  # warm
    one = min(timed(1) for _ in range(2))
    many = min(timed(tokens) for _ in range(2))
    per_step = (many - one) / (tokens - 1)
    bucket = llm.graphs.bucket_for(batch) if llm.graphs else None
    return {"value": batch / per_step, "unit": "tok/s",
            "h2d_bytes_per_step": bucket.words * 4 if bucket else 0,
            "d2h_bytes_per_step": (bucket.size if bucket else batch) * 4,
            "ms_per_step": per_step * 1000}


# ---- per-kernel times: a step with and without each kernel class --------------------------
def _timed_graph(body, repeats: int) -> float:
    """Milliseconds of one replay of ``body`` captured as a CUDA graph (best of ``repeats``;
    the body has run twice before the capture)."""
    import torch

    body()
    body()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        body()
    graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = math.inf
    for _ in range(repeats):
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize()
        best = min(best, start.elapsed_time(stop))
    del graph
    return best


def kernel_classes(cfg: dict) -> dict[str, str]:
    """Short name -> kernel class as ``ayaka_b200.kernels.ops`` names it."""
    d, f, v = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"]
    return {"qkv": f"linear:{3 * d}x{d}", "attn_out": f"linear:{d}x{d}", "fc": f"linear:{f}x{d}",
            "proj": f"linear:{d}x{f}", "head": f"linear:{v}x{d}", "layer_norm": "layer_norm"}


def profile_decode(llm, cfg: dict, batch: int, peak: dict) -> dict:
    """What each kernel class costs inside a decode step of ``batch`` requests at context
    ~530: the step's own CUDA graph body is captured again with one class left out
    (``ops.leaving_out``) and the difference of the replay times is the class's share of the
    dependent chain. ``frac`` is its bytes (weights read once, or the live keys and values)
    over that time over the measured copy bandwidth."""
    import torch

    from ayaka_b200 import SamplingParams
    from ayaka_b200.kernels import ops

    scheduler = llm.scheduler
    params = SamplingParams(temperature=0.0, max_tokens=None, ignore_eos=True)
    for index, prompt in enumerate(random_prompts(cfg, batch, PROMPT, 77)):
        scheduler.add_request(f"profile{batch}-{index}", prompt, params)
    while any(r.prefilling for r in scheduler.running.values()) or scheduler.waiting:
        llm._advance()
    for _ in range(16):
        llm._advance()
    llm.graphs.drop_ahead()
    torch.cuda.synchronize()
    context = PROMPT + 17
    bucket = llm.graphs.bucket_for(batch)
    core = llm.core

    def body() -> None:
        bucket.launch_body(core, True)

    d, f, v, layers = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"], cfg["n_layer"]
    classes = {**kernel_classes(cfg), "attention": "attention_decode", "argmax": "argmax",
               "embed": "embed_rows"}
    nbytes = {"qkv": layers * 3 * d * d * 2, "attn_out": layers * d * d * 2,
              "fc": layers * d * f * 2, "proj": layers * d * f * 2, "head": v * d * 2,
              "attention": layers * batch * context * 2 * d * 2,
              "layer_norm": (2 * layers + 1) * batch * d * 6,
              "argmax": batch * v * 4, "embed": batch * d * 8}
    full = _timed_graph(body, 10)
    out = {"step_us": round(full * 1000, 1), "context": context, "batch": batch,
           "method": "graph replay of the step with and without the class"}
    for name, klass in classes.items():
        with ops.leaving_out(klass):
            without = _timed_graph(body, 10)
        us = max(full - without, 1e-6) * 1000
        per = layers if name not in ("head", "argmax", "embed") else 1
        out[name] = {"us": round(us, 1), "per_layer_us": round(us / per, 2),
                     "bytes": nbytes[name],
                     "frac": round(nbytes[name] / (us * 1e-6) / 1e9 / peak["hbm_gbs"], 3),
                     "peak": "hbm_gbs"}
    for request_id in list(scheduler.running):
        scheduler.abort(request_id)
    scheduler.take_events()
    return out


def profile_prefill(llm, cfg: dict, peak: dict) -> dict:
    """Each kernel class inside one 2,048-token prompt step (two prompts of 1,024), two ways.
    ``alone_us``: the class's own kernels, from CUDA events around every launch of the step
    (``ops.timed``), with the device kept busy ahead of the step so that no host time falls
    between a launch's events; no kernel starts under its predecessor's tail then, so the
    sum is more than the step. ``us``: what the step loses when the class is left out
    (``ops.leaving_out``, the step replayed as a CUDA graph), i.e. the class's share of the
    chain of dependent launches; a kernel whose time hides the start-up of its neighbours
    measures little here. ``frac`` is the class's floating-point work over ``alone_us`` over
    the measured bf16 matrix-product peak; for the norms, the embedding and the head (two
    rows) its bytes over the copy bandwidth."""
    import torch

    from ayaka_b200.engine.runner import StepEntry
    from ayaka_b200.kernels import ops

    core = llm.core
    length = cfg["n_positions"]
    entries = [StepEntry(f"profile-prefill-{i}", prompt, (length - 1,))
               for i, prompt in enumerate(random_prompts(cfg, 2, length, 990))]
    d, f, v, layers = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"], cfg["n_layer"]
    tokens = 2 * length
    classes = {**kernel_classes(cfg), "attention": "attention_prefill", "embed": "embed_rows"}
    names = {klass: name for name, klass in classes.items()}
    alone: dict[str, float] = {}
    for _ in range(4):
        torch.cuda.synchronize()
        torch.cuda._sleep(40_000_000)  # about 20 ms: the launches below queue up behind it
        with ops.timed() as record:
            core.step(entries)
        torch.cuda.synchronize()
        for klass, pairs in record.items():
            total = sum(a.elapsed_time(b) for a, b in pairs) * 1000
            name = names.get(klass, klass)
            alone[name] = min(alone.get(name, math.inf), total)
        for entry in entries:
            core.release(entry.request_id)

    for entry in entries:
        if not core.manager.allocate(entry.request_id, length):
            raise RuntimeError("no room for the prefill profile")
    step, want_rows, num_want = core.runner.prepare(entries)
    torch.cuda.synchronize()

    def body() -> None:
        core.model.forward(step, core.runner.caches, want_rows, num_want)

    full = _timed_graph(body, 5)
    flops = {"qkv": 2.0 * tokens * 3 * d * d * layers, "attn_out": 2.0 * tokens * d * d * layers,
             "fc": 2.0 * tokens * d * f * layers, "proj": 2.0 * tokens * d * f * layers,
             "attention": layers * 2 * 4.0 * d * (length * (length + 1) / 2)}
    nbytes = {"layer_norm": 2 * layers * tokens * d * 6, "head": v * d * 2,
              "embed": tokens * d * 8}
    out = {"step_us": round(full * 1000, 1), "tokens": tokens,
           "alone_sum_us": round(sum(alone.values()), 1),
           "method": "alone_us: events around every launch; us: the step as a graph with "
                     "and without the class"}
    for name, klass in classes.items():
        with ops.leaving_out(klass):
            without = _timed_graph(body, 5)
        own = alone.get(name, 0.0)
        per = layers if name not in ("head", "embed") else 1
        record = {"us": round(max(full - without, 0.0) * 1000, 1), "alone_us": round(own, 1),
                  "alone_per_layer_us": round(own / per, 2)}
        if own > 0 and name in flops:
            record.update(flops=flops[name], peak="bf16_tflops (burst)",
                          frac=round(flops[name] / (own * 1e-6) / 1e12 / peak["bf16_tflops"], 3))
        elif own > 0 and name in nbytes:
            record.update(bytes=nbytes[name], peak="hbm_gbs",
                          frac=round(nbytes[name] / (own * 1e-6) / 1e9 / peak["hbm_gbs"], 3))
        out[name] = record
    for entry in entries:
        core.manager.free(entry.request_id)
    core.manager.check_integrity()
    return out


def workload_run(which: str) -> dict:
    """The two serving workloads BASELINE.json names beside the headline (``configs[3]`` and
    ``configs[4]``), through ``LLM.generate`` with host token ids in and out; one JSON line.

    ``small``: GPT-2 small sizes, 64 requests with prompt lengths uniform in [16, 1024) (cut
    so that 128 more tokens fit), 128 greedy tokens each. ``large``: GPT-2 large sizes, 32
    requests decoding 256 tokens at temperature 1.0 while eight 1,000-token prompts arrive in
    portions of 256 tokens beside them (a step's budget is 288 tokens), page size 16."""
    import torch

    from ayaka_b200 import SamplingParams

    def sized(n_layer: int, width: int, heads: int, inner: int) -> dict:
        return {**XL, "n_layer": n_layer, "n_embd": width, "n_head": heads, "n_inner": inner}

    generator = torch.Generator().manual_seed(7)

    def prompts(lengths: list[int]) -> list[tuple[int, ...]]:
        return [tuple(torch.randint(0, XL["vocab_size"], (n,), generator=generator).tolist())
                for n in lengths]

    if which == "small":
        cfg = sized(12, 768, 12, 3072)
        lengths = [min(int(n), cfg["n_positions"] - 128)
                   for n in torch.randint(16, 1024, (64,), generator=generator).tolist()]
        llm = build(cfg, 64, 2048)
        batch = prompts(lengths)
        params: object = SamplingParams(temperature=0.0, max_tokens=128, ignore_eos=True)
        name = "GPT-2 small, 64 requests, prompts of 16 to 896 tokens, 128 greedy tokens each"
    else:
        cfg = sized(36, 1280, 20, 5120)
        lengths = [64] * 32 + [1000] * 8
        llm = build(cfg, 40, 288)
        batch = prompts(lengths)
        params = [SamplingParams(temperature=1.0, max_tokens=256 if i < 32 else 8,
                                 ignore_eos=True, seed=i) for i in range(40)]
        name = ("GPT-2 large, 32 requests decoding at temperature 1.0 beside 256-token "
                "portions of eight 1,000-token prompts")
    llm.generate(batch[:4], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    best, generated = math.inf, 0
    for _ in range(3):
        begin = time.perf_counter()
        outputs = llm.generate(batch, params)
        best = min(best, time.perf_counter() - begin)
        generated = sum(len(o.outputs[0].token_ids) for o in outputs)
    del llm
    torch.cuda.empty_cache()
    return ({
        "metric": f"generated tok/s through LLM.generate ({name})", "impl": "ours",
        "value": round(generated / best, 1), "unit": "tok/s", "n_gpus": 1, "dtype": "bf16",
        "data": "synthetic", "ms": round(best * 1000, 1), "generated_tokens": generated,
        "prompt_tokens": sum(lengths),
        "config": {"n_layer": cfg["n_layer"], "n_embd": cfg["n_embd"], "n_head": cfg["n_head"],
                   "n_inner": cfg["n_inner"], "vocab_size": cfg["vocab_size"],
                   "n_positions": cfg["n_positions"], "page_size": 16,
                   "weights": "random bf16 seed 0", "cuda_graph": True}})


def config_record(cfg: dict, mean_context: float, prompt_len: int = PROMPT) -> dict:
    """The ``config`` of the line: every size, flat; the same for both arms."""
    return {
        "model": "gpt2-xl", "n_layer": cfg["n_layer"], "n_layer_full": XL["n_layer"],
        "n_embd": cfg["n_embd"], "n_head": cfg["n_head"], "n_inner": cfg["n_inner"],
        "vocab_size": cfg["vocab_size"], "n_positions": cfg["n_positions"],
        "global_batch": 8, "seq_len": cfg["n_positions"], "prompt_len": prompt_len,
        "mean_context": round(mean_context, 1), "page_size": 16,
        "parallelism": "single-gpu", "weights": "random bf16 seed 0",
        "l2": "inputs larger than L2 (3.1 GB of weights per step)", "cuda_graph": True,
    }


def reference_arm(args: argparse.Namespace) -> int:
    """The same measurement on the unmodified reference (``baseline/reference_arm.py``)."""
    sys.path.insert(0, str(ROOT / "baseline"))
    import reference_arm as arm

    return arm.run(args, {**XL, "n_layer": args.layers})


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=400)
    parser.add_argument("--warmup", type=int, default=16)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--layers", type=int, default=48,
                        help="layers to build (GPT-2 XL has 48); sizes of a layer never change")
    parser.add_argument("--batch", type=int, default=8,
                        help="requests of the headline decode run (8; other values are for "
                             "profiling a batch size under ncu)")
    parser.add_argument("--skip-points", action="store_true",
                        help="leave out the batch 1 / batch 64 points and the e2e run")
    parser.add_argument("--no-profile", action="store_true",
                        help="leave out the per-kernel times (a step with and without each "
                             "kernel class)")
    parser.add_argument("--skip-workloads", action="store_true",
                        help="leave out the two serving workloads of the other configurations")
    parser.add_argument("--workload", choices=("small", "large"),
                        help="instead of the headline run: one of the two serving workloads "
                             "(GPT-2 small with 64 ragged requests; GPT-2 large with prompt "
                             "portions beside 32 decoding requests)")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    import torch

    if not torch.cuda.is_available():
        print("bench.py: no CUDA device")
        return 1
    if args.workload:
        print(json.dumps(workload_run(args.workload)))
        return 0
    warmup = max(args.warmup, 3)
    steps = max(1, min(args.steps, XL["n_positions"] - PROMPT - 2 - warmup))
    cfg = {**XL, "n_layer": args.layers}
    peak, peak_source = peaks()

    llm = build(cfg, 64, 2048)
    clocks = Clocks()
    clocks.start()
    batch = max(1, min(args.batch, 64))
    main_run = decode_run(llm, cfg, batch, warmup, steps, seed=1)
    clock_record = clocks.stop()
    clock_record["window"] = f"prefill, warm-up and timed steps of the batch-{batch} run"
    prefill = prefill_run(llm, cfg, 2, 5)
    points, e2e, kernels, workloads = {}, None, None, None
    if not args.skip_points:
        for point in (1, 64):
            run = decode_run(llm, cfg, point, warmup, steps, seed=10 + point)
            points[f"decode_b{point}"] = round(point * 1000.0 / run["ms"], 1)
            points[f"decode_b{point}_ms"] = round(run["ms"], 4)
            points[f"decode_b{point}_context"] = round(run["mean_context"], 1)
            batch_bytes = layer_weight_bytes(cfg, cfg["n_layer"]) + \
                point * run["mean_context"] * kv_bytes_per_token(cfg, cfg["n_layer"])
            points[f"decode_b{point}_hbm_frac"] = round(
                batch_bytes / (run["ms"] * 1e-3) / 1e9 / peak["hbm_gbs"], 4)
        e2e = e2e_run(llm, cfg, batch, 128)
    if not args.no_profile:
        from ayaka_b200.kernels import ops

        # the Python forward launches the same kernels as the C++ host code, one call each,
        # which is where a kernel class can be left out or bracketed by events
        ops.NATIVE_STEP = False
        try:
            kernels = {f"decode_b{batch}": profile_decode(llm, cfg, batch, peak)}
            if batch != 64:
                kernels["decode_b64"] = profile_decode(llm, cfg, 64, peak)
            kernels["prefill_2048"] = profile_prefill(llm, cfg, peak)
        finally:
            ops.NATIVE_STEP = True
    if not args.skip_workloads:
        llm.close()
        del llm
        torch.cuda.empty_cache()
        workloads = {}
        for which in ("small", "large"):
            record = workload_run(which)
            workloads[which] = {"value": record["value"], "unit": "generated tok/s",
                                "ms": record["ms"], "generated_tokens": record["generated_tokens"],
                                "prompt_tokens": record["prompt_tokens"],
                                "what": record["metric"]}

    layers = cfg["n_layer"]
    step_bytes = layer_weight_bytes(cfg, layers) + \
        batch * main_run["mean_context"] * kv_bytes_per_token(cfg, layers)
    achieved = step_bytes / (main_run["ms"] * 1e-3) / 1e9
    flops = prefill_flops(cfg, layers, 2, cfg["n_positions"])
    value = batch * 1000.0 / main_run["ms"]
    line = {
        "metric": METRIC if batch == 8 else METRIC.replace("batch 8", f"batch {batch}"),
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {**config_record(cfg, main_run["mean_context"]), "global_batch": batch},
        "prefill": {"value": round(prefill["tokens"] * 1000.0 / prefill["ms"], 1),
                    "tokens": prefill["tokens"], "ms": round(prefill["ms"], 3),
                    "frac": round(flops / (prefill["ms"] * 1e-3) / (peak["bf16_tflops"] * 1e12),
                                  4), "peak": "bf16_tflops (burst)"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1),
                     "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "peaks": peak_source},
        "points": points,
        "clocks": clock_record,
        "gpu_launches": int(main_run["launches"]),
        "host_ms_per_step": round(main_run["wall_ms"], 4),
    }
    if e2e is not None:
        line["e2e"] = {key: (round(val, 2) if isinstance(val, float) else val)
                       for key, val in e2e.items()}
    if kernels is not None:
        line["kernels"] = kernels
    if workloads is not None:
        line["workloads"] = workloads
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
