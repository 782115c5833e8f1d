"""``forge-engine`` command line: ``generate`` and ``doctor``.

Option names and meanings follow upstream's ``chat``/``serve`` where it has them
(src/forge_engine/cli.py:38-66): --max-new-tokens, --temperature, --top-k, --top-p,
--min-p, --seed, --max-requests, --max-batch-size, --token-budget, --block-size,
--block-capacity.  ``doctor`` prints ``key=value`` lines like upstream's
(src/forge_engine/cli.py:94-127).  Upstream has no ``generate`` (it chats through a
tokenizer and serves HTTP); this engine takes and prints token ids.  Errors go to
stderr as ``forge-engine: message`` with exit code 1, as upstream does.
"""

from __future__ import annotations

import argparse
import json
import platform
import shutil
import sys
from collections.abc import Sequence

from . import __version__
from .errors import ForgeEngineError


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="forge-engine")
    parser.add_argument("--version", action="version", version=f"%(prog)s {__version__}")
    commands = parser.add_subparsers(dest="command", required=True)
    generate = commands.add_parser("generate", help="generate token ids for one or more prompts")
    source = generate.add_mutually_exclusive_group(required=True)
    source.add_argument("--model", help="folder with config.json and safetensors weights")
    source.add_argument("--random-weights", type=int, metavar="SEED",
                        help="draw random weights from SEED for the model of --config")
    generate.add_argument("--config", help="config.json to use with --random-weights")
    generate.add_argument("--save-model", metavar="DIR",
                          help="with --random-weights: also write config.json and model.safetensors to DIR")
    generate.add_argument("--prompt-ids", action="append", required=True,
                          help="comma-separated token ids; may be given more than once")
    generate.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    generate.add_argument("--device", default="cuda:0")
    generate.add_argument("--max-new-tokens", type=int, default=256)
    generate.add_argument("--temperature", type=float, default=0.0)
    generate.add_argument("--top-k", type=int)
    generate.add_argument("--top-p", type=float, default=1.0)
    generate.add_argument("--min-p", type=float, default=0.0)
    generate.add_argument("--seed", type=int)
    generate.add_argument("--max-requests", type=int, default=16)
    generate.add_argument("--max-batch-size", type=int, default=8)
    generate.add_argument("--token-budget", type=int, default=256)
    generate.add_argument("--block-size", type=int, default=16)
    generate.add_argument("--block-capacity", type=int, default=1024)
    generate.add_argument("--chunk-size", type=int)
    commands.add_parser("doctor", help="print the local engine and CUDA environment")
    return parser


def run_doctor() -> int:
    import torch

    from .ops.build import CSRC, LIB_NAME, find_nvcc

    cuda = bool(torch.cuda.is_available())
    try:
        nvcc = find_nvcc()
    except ForgeEngineError:
        nvcc = None
    built = any((d / LIB_NAME).is_file() for d in (CSRC / "_build",))
    free_memory = "unavailable"
    if cuda:
        free, total = torch.cuda.mem_get_info(0)
        free_memory = f"{free // 2**20}MiB of {total // 2**20}MiB"
    fields = (
        ("forge_engine_version", __version__),
        ("python_version", platform.python_version()),
        ("pytorch_version", torch.__version__),
        ("cuda_available", cuda),
        ("gpu_name", torch.cuda.get_device_name(0) if cuda else "unavailable"),
        ("compute_capability",
         ".".join(map(str, torch.cuda.get_device_capability(0))) if cuda else "unavailable"),
        ("bf16_supported", bool(torch.cuda.is_bf16_supported()) if cuda else False),
        ("cuda_toolkit_available", nvcc is not None),
        ("g++_available", shutil.which("g++") is not None),
        ("ninja_available", shutil.which("ninja") is not None),
        ("kernel_target", "sm_100a"),
        ("kernel_library_built", built),
        ("gpu_memory_free", free_memory),
        ("architectures", ",".join(__import__("forge_engine_b200.config", fromlist=["x"]).known_architectures())),
    )
    for name, value in fields:
        print(f"{name}={value}")
    return 0


def run_generate(args: argparse.Namespace) -> int:
    from .config import EngineConfig, SchedulerConfig
    from .engine import Engine

    prompts = []
    for text in args.prompt_ids:
        try:
            prompts.append([int(t) for t in text.replace(" ", "").split(",") if t])
        except ValueError:
            raise ValueError(f"--prompt-ids {text!r} is not a comma-separated list of integers") from None
    engine_config = EngineConfig(
        max_new_tokens=args.max_new_tokens,
        temperature=args.temperature,
        top_k=args.top_k,
        top_p=args.top_p,
        min_p=args.min_p,
        seed=args.seed,
        dtype=args.dtype,
    )
    scheduler_config = SchedulerConfig(
        max_requests=args.max_requests,
        max_batch_size=args.max_batch_size,
        token_budget=args.token_budget,
        block_size=args.block_size,
        block_capacity=args.block_capacity,
        chunk_size=args.chunk_size,
    )
    if args.model:
        engine = Engine.from_pretrained(args.model, engine_config=engine_config,
                                        scheduler_config=scheduler_config, device=args.device)
    else:
        if not args.config:
            raise ValueError("--random-weights needs --config FILE")
        with open(args.config) as handle:
            raw = json.load(handle)
        if args.save_model:
            import torch

            from .config import read_model_config
            from .weights import random_tensors, write_model_folder

            arch, _, spec = read_model_config(raw)
            write_model_folder(args.save_model, raw,
                               random_tensors(arch.expected_tensors(spec), args.random_weights, dtype=torch.bfloat16))
            engine = Engine.from_pretrained(args.save_model, engine_config=engine_config,
                                            scheduler_config=scheduler_config, device=args.device)
        else:
            engine = Engine.from_random(raw, args.random_weights, engine_config=engine_config,
                                        scheduler_config=scheduler_config, device=args.device)
    for output in engine.generate(prompts):
        print(",".join(str(t) for t in output))
    return 0


def main(argv: Sequence[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    try:
        if args.command == "doctor":
            return run_doctor()
        if args.command == "generate":
            return run_generate(args)
    except (ForgeEngineError, ValueError) as error:
        print(f"forge-engine: {error}", file=sys.stderr)
        return 1
    return 2


if __name__ == "__main__":
    raise SystemExit(main())
