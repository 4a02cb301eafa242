"""Command line of liteinfer_b200: `python -m liteinfer_b200 <command>`.

The reference ships no generation command line (its only script is the
benchmark harness, pyproject.toml:44-45); the options here carry the names of
its `EngineConfig` fields (liteinfer/config.py:13-67) and `SamplingParams` fields
(liteinfer/sampling/params.py:9-21), with dashes for underscores.

    generate        generate from prompts (text, or token ids for a model without a tokenizer)
    random-weights  write a model folder (config.json, model.safetensors) from a config and a seed
    replay          trace replay (the same program as bin/trace_run)
    bench run       throughput and latency on synthetic requests, with the option names and the summaries of the
                    reference's `bench dataset` / `bench run` (benchmarks/cli.py:209-265)
    build           compile every CUDA library now
"""

from __future__ import annotations

import argparse
import json
import sys


def _add_engine_options(parser: argparse.ArgumentParser) -> None:
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    parser.add_argument("--device", default="auto")
    parser.add_argument("--max-num-seqs", type=int, default=32)
    parser.add_argument("--max-model-len", type=int, default=4096)
    parser.add_argument("--max-num-batched-tokens", type=int, default=None)
    parser.add_argument("--block-size", type=int, default=16)
    parser.add_argument("--num-gpu-blocks", type=int, default=None)
    parser.add_argument("--gpu-memory-utilization", type=float, default=0.85)
    parser.add_argument("--paged-decode-splits", type=int, default=None)
    parser.add_argument("--enable-cuda-graphs", dest="enable_cuda_graphs", action="store_true", default=None)
    parser.add_argument("--no-cuda-graphs", dest="enable_cuda_graphs", action="store_false")
    parser.add_argument("--seed", type=int, default=42, help="engine seed (requests without a seed of their own)")


def _add_sampling_options(parser: argparse.ArgumentParser) -> None:
    parser.add_argument("--temperature", type=float, default=1.0)
    parser.add_argument("--top-p", type=float, default=1.0)
    parser.add_argument("--top-k", type=int, default=-1)
    parser.add_argument("--max-tokens", type=int, default=64)
    parser.add_argument("--min-tokens", type=int, default=0)
    parser.add_argument("--ignore-eos", action="store_true")
    parser.add_argument("--stop", action="append", default=None)
    parser.add_argument("--stop-token-ids", type=int, nargs="*", default=None)
    parser.add_argument("--sampling-seed", type=int, default=None, help="SamplingParams.seed")


def _generate(args: argparse.Namespace) -> int:
    from liteinfer_b200.engine.llm import LLM
    from liteinfer_b200.sampling.params import SamplingParams

    prompts: list = list(args.prompt or [])
    for ids in args.prompt_ids or []:
        prompts.append([int(t) for t in ids.replace(",", " ").split()])
    if not prompts:
        print("generate: give --prompt or --prompt-ids", file=sys.stderr)
        return 2
    params = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
                            max_tokens=args.max_tokens, min_tokens=args.min_tokens, ignore_eos=args.ignore_eos,
                            stop=args.stop, stop_token_ids=args.stop_token_ids, seed=args.sampling_seed)
    with LLM(args.model, dtype=args.dtype, device=args.device, max_num_seqs=args.max_num_seqs,
             max_model_len=args.max_model_len, max_num_batched_tokens=args.max_num_batched_tokens,
             block_size=args.block_size, num_gpu_blocks=args.num_gpu_blocks,
             gpu_memory_utilization=args.gpu_memory_utilization, paged_decode_splits=args.paged_decode_splits,
             enable_cuda_graphs=args.enable_cuda_graphs, seed=args.seed) as llm:
        for out in llm.generate(prompts, params):
            print(json.dumps({"request_id": out.request_id, "prompt": out.prompt, "text": out.text,
                              "token_ids": out.token_ids, "finish_reason": out.finish_reason}))
    return 0


def _random_weights(args: argparse.Namespace) -> int:
    from liteinfer_b200.config.engine_config import parse_dtype
    from liteinfer_b200.weights.random_init import write_random_model

    raw = json.loads(open(args.config).read())
    out = write_random_model(raw, args.out, args.seed, parse_dtype(args.dtype))
    print(out)
    return 0


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="liteinfer_b200", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="command", required=True)

    gen = sub.add_parser("generate", help="generate from prompts")
    gen.add_argument("--model", required=True)
    gen.add_argument("--prompt", action="append", help="a prompt as text (repeatable)")
    gen.add_argument("--prompt-ids", action="append", help="a prompt as token ids, e.g. '5 17 3' (repeatable)")
    _add_engine_options(gen)
    _add_sampling_options(gen)

    rnd = sub.add_parser("random-weights", help="write a random model folder")
    rnd.add_argument("--config", required=True, help="a config.json of the architecture")
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--out", required=True)
    rnd.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])

    sub.add_parser("replay", help="trace replay; arguments as bin/trace_run", add_help=False)
    bench = sub.add_parser("bench", help="benchmarks in the reference's manner")
    bench_sub = bench.add_subparsers(dest="bench_command", required=True)
    run = bench_sub.add_parser("run", help="make the synthetic dataset and run it")
    run.add_argument("--model", required=True)
    run.add_argument("--isl", required=True, help="tokens per prompt, or 'mixed'")
    run.add_argument("--osl", type=int, required=True, help="tokens generated per request (forced)")
    run.add_argument("--max-isl", type=int, default=2048, help="longest prompt of a mixed dataset")
    run.add_argument("-n", "--num-samples", type=int, default=200)
    run.add_argument("--mode", choices=["throughput", "latency", "both"], default="both")
    run.add_argument("--results-dir", default=None, help="also write the result as a JSON file here")
    run.add_argument("--dataset-seed", type=int, default=0)
    _add_engine_options(run)
    sub.add_parser("build", help="compile every CUDA library")

    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":
        from liteinfer_b200.replay import main as replay_main
        return replay_main(argv[1:])
    args = parser.parse_args(argv)
    if args.command == "generate":
        return _generate(args)
    if args.command == "random-weights":
        return _random_weights(args)
    if args.command == "bench":
        from liteinfer_b200.benchmark import main as bench_main
        return bench_main(args)
    if args.command == "build":
        from liteinfer_b200.ops import build_all
        for path in build_all():
            print(path)
        return 0
    return 2


if __name__ == "__main__":
    sys.exit(main())
