"""The command line: ``python -m ayaka_b200 run MODEL -p "5,17,3"``.

Flags carry the names and meanings of the reference's ``ayaka run``
(``python/ayaka/entrypoints/cli.py:162-209, 335-383``) where it has them: ``-p/--prompt``
(standard input when absent), ``--max-tokens`` (128), ``--temperature`` (0 = greedy),
``--top-k`` (-1 = off), ``--top-p`` (1), ``--seed``, ``--device``, ``--dtype``,
``--cuda-graph``, ``--memory-ratio``, ``--kv-reserve-tokens``, ``-q``, ``-v``. Prompts and
results are token ids (this engine has no tokenizer): the prompt is integers separated by
commas or spaces, the generated ids go to standard output, everything else to standard
error. Exit codes follow ``python/ayaka/entrypoints/console.py:34-41``: 0 ok, 1 bug, 2 usage,
3 model cannot be loaded, 4 model not found, 5 not enough memory, 6 engine failure, 130
interrupted. Typed errors print one line, never a traceback.

``python -m ayaka_b200 random CONFIG.json OUT`` writes a model folder with random weights;
``python -m ayaka_b200 replay --model DIR --dtype D --out DIR --max-tokens N`` is the trace
replay program (``bin/trace_run``); ``python -m ayaka_b200 info`` prints what this
installation has, after the reference's ``ayaka info`` (``entrypoints/cli.py:212-219``):
version, devices, architectures and parts it knows, compiler and compiled libraries.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

from ayaka_b200.errors import (AyakaError, BackendError, CapacityError, ConfigError,
                               InvalidRequestError, ModelLoadError)

EXIT_OK, EXIT_BUG, EXIT_USAGE, EXIT_LOAD, EXIT_MISSING, EXIT_MEMORY, EXIT_ENGINE = range(7)
EXIT_INTERRUPTED = 130
PROG = "ayaka_b200"


def say(text: str) -> None:
    print(f"{PROG}: {text}", file=sys.stderr, flush=True)


def _parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog=PROG, description="GPT-2 inference on one B200.")
    commands = parser.add_subparsers(dest="command", metavar="command")
    run = commands.add_parser("run", help="generate token ids for a prompt and print them")
    run.add_argument("model", help="a local model folder (config.json, model.safetensors)")
    run.add_argument("-p", "--prompt", help="the prompt's token ids, separated by commas or "
                     "spaces; when absent they are read from standard input")
    sampling = run.add_argument_group("sampling")
    sampling.add_argument("--max-tokens", type=int, default=128, metavar="N",
                          help="most tokens to generate (128)")
    sampling.add_argument("--temperature", type=float, default=0.0, metavar="T",
                          help="softmax temperature; 0 is greedy decoding (0)")
    sampling.add_argument("--top-k", type=int, default=-1, metavar="K", help="top-k; -1 is off")
    sampling.add_argument("--top-p", type=float, default=1.0, metavar="P", help="top-p (1)")
    sampling.add_argument("--min-p", type=float, default=0.0, metavar="P", help="min-p (0)")
    sampling.add_argument("--seed", type=int, default=None, metavar="S",
                          help="seed of the random numbers; the same seed gives the same ids")
    sampling.add_argument("--stop-token-id", type=int, action="append", default=[], metavar="ID",
                          help="stop when this token is generated (repeatable)")
    sampling.add_argument("--ignore-eos", action="store_true",
                          help="do not stop at the model's end-of-sequence token")
    where = run.add_argument_group("where and how it runs")
    where.add_argument("--device", default="cuda", metavar="DEVICE", help="cuda or cuda:N (cuda)")
    where.add_argument("--dtype", choices=("bf16", "bfloat16", "fp32", "float32"), default="fp32",
                       help="compute dtype of the model (fp32)")
    where.add_argument("--cuda-graph", action="store_true",
                       help="capture decode steps in CUDA graphs and replay them")
    where.add_argument("--memory-ratio", type=float, default=None, metavar="R",
                       help="share of the free memory the cache may use, in (0, 1] (0.9)")
    where.add_argument("--kv-reserve-tokens", type=int, default=None, metavar="N",
                       help="tokens the cache must hold; the model context when absent")
    where.add_argument("--block-size", type=int, default=16, metavar="N",
                       help="tokens per cache page (16)")
    where.add_argument("--max-tokens-per-step", type=int, default=2048, metavar="N",
                       help="token budget of one step (2048)")
    run.add_argument("-q", "--quiet", action="store_true", help="do not print the start-up line")
    run.add_argument("-v", "--verbose", action="count", default=0, help="log progress")

    commands.add_parser(
        "replay", add_help=False,
        help="feed given token ids through a model step by step and write the logits "
             "(the program bin/trace_run; `replay --help` lists its options)")
    info = commands.add_parser(
        "info", help="print the version, devices, architectures, parts and CUDA libraries")
    info.add_argument("--output", choices=("text", "json"), default="text", help="text or json")
    rand = commands.add_parser("random", help="write a model folder with random weights")
    rand.add_argument("config", help="a config.json (the architecture's own keys)")
    rand.add_argument("out", help="folder to write config.json and model.safetensors into")
    rand.add_argument("--seed", type=int, default=0)
    rand.add_argument("--dtype", choices=("bfloat16", "float32"), default="float32",
                      help="dtype the tensors are stored in (float32)")
    rand.add_argument("--weight-std", type=float, default=0.02)
    rand.add_argument("--bias-std", type=float, default=0.0)
    rand.add_argument("--norm-std", type=float, default=0.0)
    return parser


def _prompt_ids(text: str) -> list[int]:
    fields = text.replace(",", " ").split()
    if not fields:
        raise InvalidRequestError("the prompt is empty")
    try:
        return [int(field) for field in fields]
    except ValueError:
        raise InvalidRequestError(
            "the prompt must be token ids (integers separated by commas or spaces); this "
            "engine has no tokenizer") from None


def _run(args: argparse.Namespace) -> int:
    from ayaka_b200.config.engine import EngineConfig
    from ayaka_b200.engine.llm import LLM
    from ayaka_b200.sampling.params import SamplingParams

    if not Path(args.model).is_dir():
        say(f"model folder {args.model!r} does not exist")
        return EXIT_MISSING
    text = args.prompt if args.prompt is not None else sys.stdin.read()
    prompt = _prompt_ids(text)
    params = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                            min_p=args.min_p, seed=args.seed, max_tokens=args.max_tokens,
                            stop_token_ids=frozenset(args.stop_token_id),
                            ignore_eos=args.ignore_eos)
    config = EngineConfig(
        model=args.model, dtype=args.dtype, device=args.device, block_size=args.block_size,
        memory_ratio=args.memory_ratio if args.memory_ratio is not None else 0.9,
        kv_reserve_tokens=args.kv_reserve_tokens, max_running=1,
        max_tokens_per_step=args.max_tokens_per_step, cuda_graph=args.cuda_graph)
    with LLM.from_config(config) as llm:
        if not args.quiet:
            spec = llm.core.model.spec
            say(f"{Path(args.model).name}: {len(spec.layers)} layers, width {spec.hidden_size}, "
                f"{config.dtype}, {llm.core.manager.pools[0].num_usable} cache pages of "
                f"{config.block_size}")
        first = True
        for output in llm.stream(tuple(prompt), params):
            for token in output.outputs[0].token_ids:
                sys.stdout.write(("" if first else " ") + str(token))
                first = False
            sys.stdout.flush()
            if output.finished:
                sys.stdout.write("\n")
                if output.error:
                    say(output.error)
                    return EXIT_ENGINE
                if args.verbose:
                    say(f"finished: {output.outputs[0].finish_reason.value}, "
                        f"{output.usage.completion_tokens} tokens")
    return EXIT_OK


def _random(args: argparse.Namespace) -> int:
    from ayaka_b200.weights.random_init import write_random_model
    from ayaka_b200.weights.rules import RandomInit

    path = Path(args.config)
    if not path.is_file():
        say(f"{path} does not exist")
        return EXIT_MISSING
    config = json.loads(path.read_text(encoding="utf-8"))
    init = RandomInit(weight_std=args.weight_std, bias_std=args.bias_std, norm_std=args.norm_std)
    write_random_model(config, args.out, args.seed, init, store_dtype=args.dtype)
    say(f"wrote {args.out}")
    return EXIT_OK


def _info(args: argparse.Namespace) -> int:
    import torch

    import ayaka_b200
    from ayaka_b200.kernels import build
    from ayaka_b200.models.registry import supported_architectures
    from ayaka_b200.parts.base import registered_kinds

    import ayaka_b200.parts  # noqa: F401 - registers the built-in parts

    devices = []
    if torch.cuda.is_available():
        for index in range(torch.cuda.device_count()):
            properties = torch.cuda.get_device_properties(index)
            devices.append({"index": index, "name": properties.name,
                            "compute_capability": f"{properties.major}.{properties.minor}",
                            "memory_gib": round(properties.total_memory / 2 ** 30, 1),
                            "multiprocessors": properties.multi_processor_count})
    folder = build.CSRC / "_build"
    built = sorted(path.name for path in folder.glob("libayk_*.so")) if folder.is_dir() else []
    report = {
        "version": ayaka_b200.__version__,
        "torch": torch.__version__,
        "devices": devices,
        "architectures": supported_architectures(),
        "parts": {family: registered_kinds(family)
                  for family in ("mixer", "feed_forward", "norm", "position", "block",
                                 "embedding", "head")},
        "nvcc": build._nvcc(),
        "cuda_sources": build.library_names(),
        "compiled_libraries": built,
        "build_folder": str(folder),
    }
    if args.output == "json":
        print(json.dumps(report, indent=1))
        return EXIT_OK
    print(f"ayaka_b200 {report['version']} (torch {report['torch']})")
    if devices:
        for device in devices:
            print(f"device cuda:{device['index']}: {device['name']}, sm_"
                  f"{device['compute_capability'].replace('.', '')}, {device['memory_gib']} GiB, "
                  f"{device['multiprocessors']} SMs")
    else:
        print("devices: no CUDA device (this engine has no CPU path)")
    print("architectures: " + ", ".join(report["architectures"]))
    for family, kinds in report["parts"].items():
        print(f"parts/{family}: " + (", ".join(kinds) or "-"))
    print(f"nvcc: {report['nvcc'] or 'not found'}")
    print(f"CUDA sources: {', '.join(report['cuda_sources'])}")
    print(f"compiled libraries ({folder}): {len(built)}")
    return EXIT_OK


def main(argv: list[str] | None = None) -> int:
    arguments = list(sys.argv[1:] if argv is None else argv)
    if arguments[:1] == ["replay"]:  # its options are the replay program's own
        from ayaka_b200.engine.replay import main as replay_main

        try:
            return replay_main(arguments[1:])
        except SystemExit as stop:
            return int(stop.code or 0)
        except KeyboardInterrupt:
            return EXIT_INTERRUPTED
    parser = _parser()
    try:
        args = parser.parse_args(arguments)
    except SystemExit as stop:
        return int(stop.code or 0)
    if args.command is None:
        parser.print_help(sys.stderr)
        return EXIT_USAGE
    try:
        if args.command == "info":
            return _info(args)
        return _run(args) if args.command == "run" else _random(args)
    except KeyboardInterrupt:
        return EXIT_INTERRUPTED
    except (ConfigError, InvalidRequestError) as error:
        say(str(error))
        return EXIT_USAGE
    except ModelLoadError as error:
        say(str(error))
        return EXIT_LOAD
    except CapacityError as error:
        say(str(error))
        return EXIT_MEMORY
    except (BackendError, AyakaError) as error:
        say(str(error))
        return EXIT_ENGINE
