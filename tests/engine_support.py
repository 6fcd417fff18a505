"""Helpers of the engine tests: model folders in temporary places, replay schedules (the four
ways of cutting the work), and the comparison with the plain implementation."""

from __future__ import annotations

import json
import os
from pathlib import Path

import torch

import plain_gpt2 as plain
from ayaka_b200.weights.random_init import random_state, write_random_model

PAGE = 16


#: label -> largest error seen, as a fraction of the largest |logit| (printed after the run)
MEASURED: dict[str, float] = {}


def log_error(name: str, value: float) -> None:
    MEASURED[name] = max(MEASURED.get(name, 0.0), value)


def make_model(folder: Path, config: dict, seed: int, init, dtype: str) -> tuple[Path, dict]:
    """Write a random model folder stored in ``dtype`` and return it with the state the plain
    implementation must use: the stored values widened to float32."""
    write_random_model(config, folder, seed, init, store_dtype=dtype)
    state = random_state(config, seed, init, store_dtype=dtype)
    return folder, {name: tensor.float() for name, tensor in state.items()}


def build_core(model_dir: Path, dtype: str, *, num_blocks: int, max_running: int = 4,
               max_tokens_per_step: int = 1024, block_size: int = PAGE, poison: bool = True):
    from ayaka_b200.config.engine import EngineConfig
    from ayaka_b200.engine.core import EngineCore

    config = EngineConfig(model=str(model_dir), dtype=dtype, block_size=block_size,
                          num_blocks=num_blocks, max_running=max_running,
                          max_tokens_per_step=max_tokens_per_step)
    return EngineCore.from_config(config, poison_cache=poison)


# ---- schedules: lists of steps; a step = (entries [(id, tokens, want)], end [ids]) -----------
def schedule_whole(sequences: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole, one step each."""
    return [{"entries": [{"id": rid, "tokens": tokens, "want": list(range(len(tokens)))}],
             "end": [rid]} for rid, tokens in sequences.items()]


def schedule_tail(sequences: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, tokens in sequences.items():
        head = max(1, len(tokens) - tail)
        steps.append({"entries": [{"id": rid, "tokens": tokens[:head],
                                   "want": list(range(head))}], "end": []})
        for index in range(head, len(tokens)):
            steps.append({"entries": [{"id": rid, "tokens": tokens[index:index + 1],
                                       "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    return steps


def schedule_portions(sequences: dict[str, list[int]],
                      sizes: tuple[int, ...] = (2, 17, 3, 16, 5, 33, 2, 64, 1, 15)) -> list[dict]:
    """Each request alone, in portions of changing size, down to two tokens (and one)."""
    steps = []
    turn = 0
    for rid, tokens in sequences.items():
        at = 0
        while at < len(tokens):
            size = min(sizes[turn % len(sizes)], len(tokens) - at)
            turn += 1
            steps.append({"entries": [{"id": rid, "tokens": tokens[at:at + size],
                                       "want": list(range(size))}], "end": []})
            at += size
        steps[-1]["end"] = [rid]
    return steps


def schedule_mixed(sequences: dict[str, list[int]], pool_tokens: int, live_limit: int = 4,
                   decode_tail: int = 6,
                   sizes: tuple[int, ...] = (5, 2, 19, 3, 32, 7, 16, 2)) -> list[dict]:
    """Up to ``live_limit`` live requests: portions of some beside single tokens of others.

    A request is admitted when the pool (``pool_tokens``, counted with each request rounded
    up to 64) has room for all of it, so the replay never runs out of pages, and requests
    that end give their pages to later ones."""
    def rounded(n: int) -> int:
        return -(-n // 64) * 64

    waiting = list(sequences.items())
    live: dict[str, int] = {}  # id -> tokens fed so far
    held = 0
    steps = []
    turn = 0
    while waiting or live:
        while waiting and len(live) < live_limit and \
                held + rounded(len(waiting[0][1])) <= pool_tokens:
            rid, tokens = waiting.pop(0)
            live[rid] = 0
            held += rounded(len(tokens))
        if not live:
            raise AssertionError("the pool cannot hold the next request")
        entries, end = [], []
        for position, rid in enumerate(list(live)):
            tokens, done = sequences[rid], live[rid]
            if (turn + position) % 5 == 4 and len(live) > 1:
                continue  # this request sits the step out and goes on later
            remaining = len(tokens) - done
            if remaining <= decode_tail:
                size = 1
            else:
                size = min(sizes[(turn + position) % len(sizes)], remaining - decode_tail)
            entries.append({"id": rid, "tokens": tokens[done:done + size],
                            "want": list(range(size))})
            live[rid] = done + size
            if live[rid] == len(tokens):
                end.append(rid)
        for rid in end:
            held -= rounded(len(sequences[rid]))
            del live[rid]
        turn += 1
        if entries:
            steps.append({"entries": entries, "end": end})
    return steps


def number(steps: list[dict]) -> list[dict]:
    return [{"step": index, **step} for index, step in enumerate(steps)]


def peak_tokens(steps: list[dict], sequences: dict[str, list[int]]) -> int:
    """The most tokens live requests hold at any time, each rounded up to 64."""
    held: dict[str, int] = {}
    peak = 0
    for step in steps:
        for entry in step["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        peak = max(peak, sum(-(-n // 64) * 64 for n in held.values()))
        for rid in step["end"]:
            del held[rid]
    return peak


# ---- running a schedule in process -----------------------------------------------------------
def replay(core, steps: list[dict]) -> dict[str, torch.Tensor]:
    """Drive ``core.step`` with the schedule and gather, per request, logits [T, vocab]."""
    from ayaka_b200.engine.runner import StepEntry

    rows: dict[str, list[torch.Tensor]] = {}
    for step in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in step["entries"]]
        logits = core.step(entries)
        core.runner.check_device_flags()
        at = 0
        for entry in step["entries"]:
            count = len(entry["want"])
            assert entry["want"] == list(range(len(entry["tokens"])))
            rows.setdefault(entry["id"], []).append(logits[at:at + count].cpu())
            at += count
        for rid in step["end"]:
            core.release(rid)
        core.manager.check_integrity()
    return {rid: torch.cat(parts) for rid, parts in rows.items()}


def plain_logits(state: dict, config: dict, sequences: dict[str, list[int]]
                 ) -> dict[str, torch.Tensor]:
    wide = plain.cast_state(state, torch.float64)
    return {rid: plain.logits(wide, config, torch.tensor(tokens)).float()
            for rid, tokens in sequences.items()}


def rounded_logits(state: dict, config: dict, sequences: dict[str, list[int]],
                   round_weights: bool = False) -> dict[str, torch.Tensor]:
    """What a bfloat16 engine should give: the plain implementation with bfloat16 roundings
    between its parts (``plain_rounded.py``), computed in float64."""
    import plain_rounded

    wide = plain.cast_state(state, torch.float64)
    return {rid: plain_rounded.logits(wide, config, torch.tensor(tokens), round_weights).float()
            for rid, tokens in sequences.items()}


# The bfloat16 engine against the plain implementation that rounds where the engine does
# (``plain_rounded.py``). What is left between the two is not a fault: the tensor-core
# attention kernels round their attention weights exp(s - reference) to bfloat16 relative to
# a running reference, so every weight is rounded differently from any oracle's (that alone
# moves single logits of these loud models by 6e-3 to 8e-3 of the scale and a row's
# root-mean-square by 1.3e-3: ``test_plain.py`` measures it on the plain implementation
# itself); a rounding that falls on the other side of a tie is rare but lands on a sensitive
# key now and then; the activation's tanh is the hardware's approximation. Rare large single
# errors and a small error everywhere are told apart: every position's root-mean-square
# error over the vocabulary must stay within 5e-3 of the logit scale (measured: 1.1e-3 to
# 3.1e-3), which a fault that moves a row by one per cent breaks, and no single logit may
# be off by more than 1.5e-2 (measured: up to 1.0e-2), half of what the float64 comparison
# has to allow. Decode-only runs have no rounded attention weights and get tighter limits
# (measured 4.2e-3 and 1.3e-3).
ROUNDED_TOLERANCE = (1.5e-2, 1.5e-2)
ROUNDED_ROW_RMS = 5e-3
DECODE_ROUNDED_TOLERANCE = (6e-3, 6e-3)
DECODE_ROUNDED_ROW_RMS = 2.5e-3


def tolerance(dtype: str) -> tuple[float, float]:
    """(rtol, atol relative to the largest |logit|) of engine vs plain implementation.

    float32: products and sums in fp32 in another order than the float64 oracle; observed
    errors are a few 1e-6 of the largest logit. bfloat16: weights are the same bf16 values
    on both sides, but the engine rounds activations to bf16 between kernels (8 mantissa
    bits, 2^-9 relative per rounding, a few dozen roundings deep)."""
    return (1e-4, 1e-4) if dtype == "float32" else (3e-2, 3e-2)


def assert_logits_close(got: dict[str, torch.Tensor], expected: dict[str, torch.Tensor],
                        dtype: str, label: str, limits: tuple[float, float] | None = None,
                        page: int = PAGE, row_rms: float | None = None) -> None:
    """Every logit within ``atol`` (a fraction of the request's largest |logit|) plus ``rtol``
    of its own size; with ``row_rms`` also every position's root-mean-square error over the
    vocabulary within that fraction of the scale (a fault that moves a whole row a little
    shows there long before it shows in the largest single error)."""
    rtol, atol_rel = limits or tolerance(dtype)
    assert set(got) == set(expected)
    worst, worst_rms = 0.0, 0.0
    for rid, want in expected.items():
        have = got[rid]
        assert have.shape == want.shape, (rid, have.shape, want.shape)
        assert torch.isfinite(have).all(), f"{label}: request {rid} has non-finite logits"
        scale = float(want.abs().max())
        error = (have - want).abs()
        worst = max(worst, float(error.max()) / scale)
        rms = (error * error).mean(dim=1).sqrt() / scale
        worst_rms = max(worst_rms, float(rms.max()))
        bad = (error > atol_rel * scale + rtol * want.abs()).any(dim=1)
        if row_rms is not None:
            bad = bad | (rms > row_rms)
        if bad.any():
            first = int(torch.nonzero(bad)[0])
            raise AssertionError(
                f"{label}: request {rid} first differs at position {first} "
                f"(page {first // page}, slot {first % page}): max error "
                f"{float(error[first].max()):.3e}, rms {float(rms[first]) * scale:.3e} of scale "
                f"{scale:.3e}")
    suffix = "/rounded-oracle" if limits else ""
    log_error(f"{label}/{dtype}{suffix}", worst)
    log_error(f"{label}/{dtype}{suffix}/row-rms", worst_rms)


def write_trace(path: Path, steps: list[dict]) -> None:
    path.write_text("".join(json.dumps(step) + "\n" for step in number(steps)), encoding="utf-8")


def run_trace_program(model_dir: Path, dtype: str, steps: list[dict], max_tokens: int,
                      out: Path, vocab: int) -> dict[str, torch.Tensor]:
    """Run ``bin/trace_run`` as a child process and read back what it wrote."""
    import subprocess
    import sys

    import numpy as np

    program = Path(__file__).resolve().parent.parent / "bin" / "trace_run"
    text = "".join(json.dumps(step) + "\n" for step in number(steps))
    done = subprocess.run(
        [sys.executable, str(program), "--model", str(model_dir), "--dtype", dtype, "--out",
         str(out), "--max-tokens", str(max_tokens)],
        input=text, capture_output=True, text=True, timeout=600, env={**os.environ})
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [line for line in done.stdout.splitlines() if line.startswith("done ")]
    assert lines == [f"done {index}" for index in range(len(steps))]
    rows: dict[str, list[torch.Tensor]] = {}
    for index, step in enumerate(steps):
        wanted = sum(len(e["want"]) for e in step["entries"])
        if not wanted:
            continue
        data = torch.from_numpy(np.fromfile(out / f"{index}.f32", dtype="<f4").reshape(
            wanted, vocab))
        at = 0
        for entry in step["entries"]:
            rows.setdefault(entry["id"], []).append(data[at:at + len(entry["want"])])
            at += len(entry["want"])
    return {rid: torch.cat(parts) for rid, parts in rows.items()}
