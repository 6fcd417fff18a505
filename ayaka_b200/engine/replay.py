"""The replay program behind ``bin/trace_run``.

It owns no forward pass, cache or loader: it builds an :class:`EngineCore` exactly as
generation does and calls its ``step`` with the tokens each line brings. The cache pool is
sized for ``--max-tokens`` tokens (each live request's count rounded up to the page size,
which is 16, so a caller that rounds to 64 is always covered), so that pages are reused.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

__all__ = ["main"]


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__)
    parser.add_argument("--model", required=True, help="folder with config.json and "
                        "model.safetensors")
    parser.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time")
    parser.add_argument("--block-size", type=int, default=16, help="tokens per cache page (16)")
    parser.add_argument("--max-running", type=int, default=4,
                        help="most requests live at a time: rows of the block table (4)")
    parser.add_argument("--max-tokens-per-step", type=int, default=None,
                        help="largest step; default: --max-tokens")
    args = parser.parse_args(argv)

    import numpy as np
    import torch

    from ayaka_b200.config.engine import EngineConfig
    from ayaka_b200.engine.core import EngineCore
    from ayaka_b200.engine.runner import StepEntry
    from ayaka_b200.errors import AyakaError

    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    page = args.block_size
    num_blocks = -(-args.max_tokens // page) + 1
    try:
        config = EngineConfig(
            model=args.model, dtype=args.dtype, block_size=page, num_blocks=num_blocks,
            max_running=max(1, min(args.max_running, num_blocks - 1)),
            max_tokens_per_step=max(args.max_tokens_per_step or args.max_tokens, page))
        core = EngineCore.from_config(config)
    except AyakaError as error:
        print(f"trace_run: {error}", file=sys.stderr)
        return 3

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        try:
            record = json.loads(line)
            number = record["step"]
            entries = [StepEntry(str(item["id"]), list(item["tokens"]),
                                 list(item.get("want", ())))
                       for item in record.get("entries", ())]
            logits = core.step(entries) if entries else None
            if logits is not None and logits.shape[0]:
                data = logits.to("cpu").numpy().astype("<f4", copy=False)
                np.ascontiguousarray(data).tofile(out / f"{number}.f32")
            else:
                torch.cuda.synchronize()
            core.runner.check_device_flags()
            for request_id in record.get("end", ()):
                core.release(str(request_id))
        except AyakaError as error:
            print(f"trace_run: step {record.get('step') if isinstance(record, dict) else '?'}"
                  f": {error}", file=sys.stderr)
            return 6
        except (KeyError, TypeError, ValueError) as error:
            print(f"trace_run: malformed step line: {error}", file=sys.stderr)
            return 2
        print(f"done {number}", flush=True)
    return 0
