"""The reference arm of ``bench.py``: the same measurement on the unmodified reference engine.

``bench.py --impl reference`` lands here. The reference (gityuko-hb/ayaka, pure Python over
torch ops) is expected as the package ``ayaka`` under ``baseline/_ref``; it is driven through
its own public API and stock code path: ``LLM.from_config(EngineConfig(...))`` on ``cuda``
in bf16 with its ``torch`` ops backend and CUDA graphs on, its token-id-only tokenizer mode
(``skip_tokenizer_init``: prompts are tuples of token ids, ``python/ayaka/core/request.py:69``),
``LLM.generate`` for the end-to-end figures and ``EngineCore.step`` for the device-timed ones.
Nothing of this repository's engine or kernels runs in this process: the model folder with
random GPT-2 XL weights is written by a child process (``python -m ayaka_b200 random``), and
the reference loads that folder as it loads any checkpoint.

The measurement is the one ``bench.py`` makes for this engine: eight 512-token prompts are
prefilled, W untimed and K timed decode steps follow (CUDA events around the K steps);
``e2e`` is (time of T tokens - time of 1 token) / (T - 1) through ``LLM.generate``, which is
how the reference times decoding itself (``benchmarks/e2e/decode.py:1-10``); ``prefill`` is two
prompts in one step (1,023 tokens each: the reference refuses a prompt that leaves no room
for one generated token, ``python/ayaka/scheduler/scheduler.py:536-550``); ``points`` are batch
1 and 64. When the package is absent or cannot run here the line says ``unavailable`` and why.
"""

from __future__ import annotations

import json
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
    return 0


def write_model(cfg: dict, folder: Path) -> Path:
    """Random weights as a checkpoint folder, written by a child process of this repository's
    ``random`` command (seed 0, stored in bfloat16): the same tensors ``bench.py`` builds its
    own engine from."""
    folder.mkdir(parents=True, exist_ok=True)
    config_path = folder / "bench_config.json"
    config_path.write_text(json.dumps(cfg))
    model = folder / "model"
    subprocess.run([sys.executable, "-m", "ayaka_b200", "random", str(config_path), str(model),
                    "--seed", "0", "--dtype", "bfloat16"], cwd=str(ROOT), check=True,
                   stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    return model


def build(model: Path, device: str, dtype_name: str, running: int, tokens_per_step: int,
          graphs: bool):
    from ayaka.configs.cache import CacheConfig
    from ayaka.configs.device import DeviceConfig
    from ayaka.configs.engine import EngineConfig
    from ayaka.configs.model_source import ModelSourceConfig
    from ayaka.configs.scheduler import SchedulerConfig
    from ayaka.configs.tokenizer import tokenizer_config_from_source
    from ayaka.engine.llm import LLM
    from ayaka.utils.dtypes import DType

    source = ModelSourceConfig(str(model), offline=True)
    buckets = tuple(sorted({1, 8, running}))
    config = EngineConfig(
        source=source,
        tokenizer=tokenizer_config_from_source(source, skip_tokenizer_init=True),
        device=DeviceConfig(device=device, dtype=DType.from_str(dtype_name), backends=("torch",),
                            cuda_graph=graphs, graph_buckets=buckets),
        cache=CacheConfig(block_size=16, prefix_cache=False),
        scheduler=SchedulerConfig(max_running=running, max_tokens_per_step=tokens_per_step))
    return LLM.from_config(config)


def greedy(max_tokens: int):
    from ayaka.core.params import SamplingParams

    return SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True)


def decode_run(llm, prompts, warmup: int, steps: int, tag: str, on_cuda: bool) -> dict:
    """Device milliseconds per decode step: the prompts are prefilled through the engine's own
    step loop until each request has its first token, then ``warmup`` untimed and ``steps``
    timed ``EngineCore.step`` calls follow (every one a decode step for all requests: the
    reference's scheduler never mixes prompt portions with decode rows)."""
    import torch

    from ayaka.core.request import GenerateRequest

    engine = llm.engine
    # room to the end of the context: with many requests the first ones decode while the
    # last ones are still being prefilled (the scheduler lets a decode step in after two
    # prefill steps), so they are a few tokens ahead when the timed steps begin
    total = llm.info.max_model_len - len(prompts[0])
    ids = [f"bench-{tag}-{index}" for index in range(len(prompts))]
    for request_id, prompt in zip(ids, prompts):
        engine.add_request(GenerateRequest(request_id=request_id, prompt=tuple(prompt),
                                           sampling=greedy(total)), stream=True)
    produced = dict.fromkeys(ids, 0)

    def advance() -> None:
        for output in engine.step():
            if output.error is not None:
                raise RuntimeError(f"a request failed: {output.error}")
            if output.request_id in produced:
                produced[output.request_id] += sum(len(o.token_ids) for o in output.outputs)

    while min(produced.values()) < 1:
        advance()
    for _ in range(warmup):
        advance()
    before = dict(produced)
    if on_cuda:
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
    wall = time.perf_counter()
    for _ in range(steps):
        advance()
    if on_cuda:
        stop.record()
        torch.cuda.synchronize()
    wall = (time.perf_counter() - wall) * 1000.0 / steps
    ms = start.elapsed_time(stop) / steps if on_cuda else wall
    if any(produced[i] - before[i] != steps for i in ids):
        raise RuntimeError(f"{tag}: a timed step was not a decode step for every request "
                           f"(tokens per request in {steps} steps: "
                           f"{sorted({produced[i] - before[i] for i in ids})})")
    for request_id in ids:
        engine.abort(request_id)
    while engine.has_unfinished:
        engine.step()
    ahead = sum(before.values()) / len(before)  # tokens each request had made, on average
    return {"ms": ms, "wall_ms": wall,
            "mean_context": len(prompts[0]) + ahead + (steps - 1) / 2}


def timed_generate(llm, prompts, max_tokens: int) -> float:
    begin = time.perf_counter()
    outputs = llm.generate([tuple(p) for p in prompts], greedy(max_tokens))
    elapsed = time.perf_counter() - begin
    for output in outputs:
        if output.error is not None:
            raise RuntimeError(f"a request failed: {output.error}")
        if len(output.outputs[0].token_ids) != max_tokens:
            raise RuntimeError("a request ended early")
    return elapsed


def run(args, cfg: dict, device: str = "cuda", dtype_name: str = "bf16",
        prompt_len: int | None = None) -> int:
    if not (REF / "ayaka" / "__init__.py").is_file():
        return unavailable(
            "the reference package is not under baseline/_ref (its build backend, hatchling, is "
            "not installable offline; copy python/ayaka of gityuko-hb/ayaka there)")
    sys.path.insert(0, str(REF))
    sys.path.insert(0, str(ROOT))
    import bench

    try:
        import torch

        import ayaka  # noqa: F401
        from ayaka.engine.llm import LLM  # noqa: F401
    except Exception as exc:  # the box lacks something the reference imports
        return unavailable(f"{type(exc).__name__}: {exc}")
    on_cuda = device.startswith("cuda")
    if on_cuda and not torch.cuda.is_available():
        return unavailable("no CUDA device")
    prompt_len = prompt_len or bench.PROMPT
    warmup = max(args.warmup, 3)
    steps = max(1, min(args.steps, cfg["n_positions"] - prompt_len - 2 - warmup))
    peak, peak_source = bench.peaks()
    try:
        with tempfile.TemporaryDirectory() as scratch:
            model = write_model(cfg, Path(scratch))
            llm = build(model, device, dtype_name, 64, 2048, graphs=on_cuda)
        with llm:
            clocks = bench.Clocks()
            clocks.start()
            main_run = decode_run(llm, bench.random_prompts(cfg, 8, prompt_len, 1), warmup,
                                  steps, "b8", on_cuda)
            clock_record = clocks.stop()
            length = cfg["n_positions"] - 1
            long_prompts = bench.random_prompts(cfg, 2, length, 900)
            timed_generate(llm, long_prompts, 1)
            prefill_ms = sorted(timed_generate(llm, bench.random_prompts(cfg, 2, length, 901 + i),
                                               1) for i in range(3))[1] * 1000.0
            points = {}
            if not args.skip_points:
                for batch in (1, 64):
                    point = decode_run(llm, bench.random_prompts(cfg, batch, prompt_len,
                                                                 10 + batch),
                                       warmup, steps, f"b{batch}", on_cuda)
                    points[f"decode_b{batch}"] = round(batch * 1000.0 / point["ms"], 1)
                    points[f"decode_b{batch}_ms"] = round(point["ms"], 4)
                    points[f"decode_b{batch}_context"] = round(point["mean_context"], 1)
            tokens = 128 if cfg["n_positions"] - prompt_len > 128 else 8
            e2e_prompts = bench.random_prompts(cfg, 8, prompt_len, 4242)
            timed_generate(llm, e2e_prompts, 4)
            one = min(timed_generate(llm, e2e_prompts, 1) for _ in range(2))
            many = min(timed_generate(llm, e2e_prompts, tokens) for _ in range(2))
            per_step = (many - one) / (tokens - 1)
    except Exception as exc:
        return unavailable(f"the reference did not run here: {type(exc).__name__}: {exc}")

    layers = cfg["n_layer"]
    step_bytes = bench.layer_weight_bytes(cfg, layers) + \
        8 * main_run["mean_context"] * bench.kv_bytes_per_token(cfg, layers)
    achieved = step_bytes / (main_run["ms"] * 1e-3) / 1e9
    flops = bench.prefill_flops(cfg, layers, 2, length)
    line = {
        "metric": bench.METRIC, "value": round(8 * 1000.0 / main_run["ms"], 1),
        "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if dtype_name == "bf16" else dtype_name,
        "data": "synthetic", "impl": "reference",
        "config": bench.config_record(cfg, main_run["mean_context"], prompt_len),
        "prefill": {"value": round(2 * length * 1000.0 / prefill_ms, 1), "tokens": 2 * length,
                    "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4),
                    "peak": "bf16_tflops (burst)", "timed": "LLM.generate of one token, wall"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peak["hbm_gbs"], 4),
                     "peaks": peak_source},
        "points": points, "clocks": clock_record,
        "gpu_launches": 0,
        "host_ms_per_step": round(main_run["wall_ms"], 4),
        "e2e": {"value": round(8 / per_step, 2), "unit": "tok/s",
                "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                "ms_per_step": round(per_step * 1000, 4),
                "note": "the reference's own LLM.generate copies its step inputs and reads the "
                        "chosen ids back every step; this arm does not count those bytes"},
        "reference": {"package": "baseline/_ref/ayaka", "backend": "torch", "cuda_graph": on_cuda,
                      "tokenizer": "skip_tokenizer_init (token ids in and out)"},
    }
    print(json.dumps(line))
    return 0
