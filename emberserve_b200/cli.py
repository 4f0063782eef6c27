"""Command line: ``python -m emberserve_b200 generate ...`` and ``... random-weights ...``.

``generate`` keeps the reference's option names and meanings (``emberserve/cli.py:12-66,
151-160,206-223``): ``--model``, ``--dtype``, ``--device``, ``--block-size``,
``--num-blocks``, ``--max-num-seqs``, ``--max-num-batched-tokens`` (default 8192, or 2048
with chunked prefill, ``cli.py:108-110``), ``--max-model-len``,
``--enable-chunked-prefill`` / ``--no-chunked-prefill``, ``--prompt``, ``--max-tokens``,
``--temperature`` (0 = greedy), ``--top-p``, ``--top-k``, ``--seed``; it prints the text
and, on standard error, ``[n tokens in t s, tok/s, finish=...]``.  Added here:
``--prompt-ids 1,2,3`` (no tokenizer needed) and ``--repetition-penalty``.  Options of
parts this engine does not have (server, quantization, tensor parallelism, speculative
decoding, prefix caching) are absent.

``random-weights`` writes a model folder (config.json, model.safetensors) from a
config.json and a seed.
"""

from __future__ import annotations

import argparse
import json
import sys
import time


def _add_engine_args(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model", required=True, help="model folder: config.json + *.safetensors")
    p.add_argument("--dtype", choices=["float32", "bfloat16"], default="bfloat16",
                   help="bfloat16: the serving kernels; float32: the true 32-bit path")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    p.add_argument("--num-blocks", type=int, default=None, help="cache pages (default: from free memory)")
    p.add_argument("--max-num-seqs", type=int, default=256)
    p.add_argument("--max-num-batched-tokens", type=int, default=None,
                   help="token budget of a step (default 8192; 2048 with chunked prefill)")
    p.add_argument("--max-model-len", type=int, default=4096)
    p.add_argument("--enable-chunked-prefill", dest="enable_chunked_prefill", action="store_true",
                   default=True, help="mix decode tokens and prompt portions in every step (default)")
    p.add_argument("--no-chunked-prefill", dest="enable_chunked_prefill", action="store_false")
    p.add_argument("--enable-cuda-graphs", dest="enable_cuda_graphs", action="store_true", default=True,
                   help="replay decode steps from CUDA graphs (default)")
    p.add_argument("--no-cuda-graphs", dest="enable_cuda_graphs", action="store_false")
    p.add_argument("--attn-backend", choices=["auto", "mma", "generic"], default="auto",
                   help="attention kernels of the bfloat16 path: the fastest that takes the case, the mma.sync "
                        "kernels only, or the 32-bit CUDA-core kernel everywhere")
    p.add_argument("--tiled-weight-copies", choices=["auto", "on", "off"], default="auto",
                   help="a second, tiled copy of the projection weights for the decode kernels: faster decode "
                        "steps for the weights' size again (auto: where that is at most a tenth of the memory)")
    p.add_argument("--debug-scratch-guard", type=int, default=0, metavar="N",
                   help="debugging: N guard elements around every scratch buffer, checked after each step")
    p.add_argument("--async-scheduling", dest="async_scheduling", action="store_true", default=True,
                   help="launch a step before the tokens of the step before it are read (default)")
    p.add_argument("--no-async-scheduling", dest="async_scheduling", action="store_false",
                   help="read every step's tokens before the next step is planned")


def engine_config_from_args(args: argparse.Namespace):
    from emberserve_b200.config.engine import EngineConfig, dtype_from_str

    budget = args.max_num_batched_tokens
    if budget is None:
        budget = 2048 if args.enable_chunked_prefill else 8192
    return EngineConfig(model_dir=args.model, device=args.device, dtype=dtype_from_str(args.dtype),
                        block_size=args.block_size, num_gpu_blocks=args.num_blocks,
                        max_num_seqs=args.max_num_seqs, max_num_batched_tokens=budget,
                        max_model_len=args.max_model_len,
                        enable_chunked_prefill=args.enable_chunked_prefill,
                        enable_cuda_graphs=args.enable_cuda_graphs,
                        async_scheduling=args.async_scheduling,
                        debug_scratch_guard=args.debug_scratch_guard, attn_backend=args.attn_backend,
                        tiled_weight_copies={"auto": None, "on": True, "off": False}[args.tiled_weight_copies])


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="emberserve_b200")
    sub = parser.add_subparsers(dest="command", required=True)
    gen = sub.add_parser("generate", help="generate a completion for one prompt")
    _add_engine_args(gen)
    group = gen.add_mutually_exclusive_group(required=True)
    group.add_argument("--prompt", help="text (the model folder must hold a tokenizer.json)")
    group.add_argument("--prompt-ids", help="comma-separated token ids")
    gen.add_argument("--chat", action="store_true", help="wrap the prompt as a user chat turn")
    gen.add_argument("--max-tokens", type=int, default=128)
    gen.add_argument("--temperature", type=float, default=0.0)
    gen.add_argument("--top-p", type=float, default=1.0)
    gen.add_argument("--top-k", type=int, default=-1)
    gen.add_argument("--repetition-penalty", type=float, default=1.0)
    gen.add_argument("--seed", type=int, default=None)

    rnd = sub.add_parser("random-weights", help="write a model folder with seeded random weights")
    rnd.add_argument("--config", required=True, help="a config.json of a supported architecture")
    rnd.add_argument("--out", required=True, help="folder to write config.json and model.safetensors to")
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--std", type=float, default=0.02)
    rnd.add_argument("--bias-std", type=float, default=0.02)
    rnd.add_argument("--store-dtype", choices=["bfloat16", "float32"], default="bfloat16")
    return parser


def cmd_generate(args: argparse.Namespace) -> int:
    from emberserve_b200.llm import LLM
    from emberserve_b200.sampling.params import SamplingParams

    llm = LLM(args.model, engine_config_from_args(args))
    params = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature,
                            top_p=args.top_p, top_k=args.top_k,
                            repetition_penalty=args.repetition_penalty, seed=args.seed)
    prompt = args.prompt if args.prompt is not None else [int(t) for t in args.prompt_ids.split(",") if t.strip()]
    if args.chat and args.prompt is None:
        raise SystemExit("--chat needs --prompt (text)")
    t0 = time.perf_counter()
    if args.chat:
        res = llm.chat([[{"role": "user", "content": args.prompt}]], params)[0]
    else:
        res = llm.generate([prompt], params)[0]
    dt = time.perf_counter() - t0
    n = len(res.output_token_ids)
    print(res.text if res.text else " ".join(str(t) for t in res.output_token_ids))
    print(f"\n[{n} tokens in {dt:.2f}s, {n / dt:.1f} tok/s, finish={res.finish_reason}]", file=sys.stderr)
    return 0


def cmd_random_weights(args: argparse.Namespace) -> int:
    from emberserve_b200.config.engine import dtype_from_str
    from emberserve_b200.registry import resolve_architecture
    from emberserve_b200.weights.loader import write_random_model

    with open(args.config) as f:
        cfg = json.load(f)
    config = resolve_architecture(cfg).config_cls.from_dict(cfg)
    out = write_random_model(config, args.out, args.seed, args.std, args.bias_std,
                             dtype_from_str(args.store_dtype))
    print(out)
    return 0


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    return cmd_generate(args) if args.command == "generate" else cmd_random_weights(args)


if __name__ == "__main__":
    sys.exit(main())
