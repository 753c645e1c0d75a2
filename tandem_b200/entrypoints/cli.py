"""Command line: ``tandem generate | replay | random-model``.

``generate`` keeps the option names and defaults of 12vivi/tandem's CLI
(python/tandem/entrypoints/cli.py:12-46,162-170) where the option still means something here;
``--prompt`` takes text when the model folder has a tokenizer, ``--prompt-ids`` takes token ids.
``replay`` is trace replay (the same program as ``bin/trace_run``); ``random-model`` writes a
model folder with seeded random weights.
"""

from __future__ import annotations

import argparse
import json
import sys
import time


def _engine_args(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model", required=True, help="model folder (config.json + *.safetensors)")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--dtype", default="auto", choices=["auto", "bfloat16", "float32"])
    p.add_argument("--max-num-seqs", type=int, default=64)
    p.add_argument("--max-num-batched-tokens", type=int, default=2048)
    p.add_argument("--schedule-policy", choices=["prefill_first", "decode_first"], default="prefill_first")
    p.add_argument("--max-model-len", type=int, default=None)
    p.add_argument("--block-size", type=int, default=16)
    p.add_argument("--kv-cache-gb", type=float, default=1.0)
    p.add_argument("--num-kv-blocks", type=int, default=None)
    p.add_argument("--no-cuda-graph", action="store_true", help="run decode steps without CUDA graphs")
    p.add_argument("--no-overlap", action="store_true", help="read every step's tokens before the next step is launched")
    p.add_argument("--cuda-graph-max-bs", type=int, default=64)
    p.add_argument("--cuda-graph-capture-at-start", action="store_true", help="capture every CUDA graph when the engine is built, not at its first use")
    p.add_argument("--no-small-batch-gemv", action="store_true", help="keep cuBLAS for every bfloat16 product, the decoder projections at small batch too")
    p.add_argument("--engine-seed", type=int, default=0, help="seed of requests that carry none")


def _engine_config(args):
    from tandem_b200.config.engine_config import EngineConfig

    return EngineConfig(
        model=args.model, device=args.device, dtype=args.dtype, max_num_seqs=args.max_num_seqs,
        max_num_batched_tokens=args.max_num_batched_tokens, schedule_policy=args.schedule_policy,
        max_model_len=args.max_model_len, block_size=args.block_size, kv_cache_memory_gb=args.kv_cache_gb,
        num_kv_blocks=args.num_kv_blocks, seed=args.engine_seed, cuda_graph=not args.no_cuda_graph, overlap_schedule=not args.no_overlap,
        cuda_graph_max_bs=args.cuda_graph_max_bs, cuda_graph_capture_at_start=args.cuda_graph_capture_at_start, small_batch_gemv=not args.no_small_batch_gemv,
    )


def cmd_generate(args) -> None:
    from tandem_b200.engine.llm_engine import LLMEngine
    from tandem_b200.sampling.params import SamplingParams

    engine = LLMEngine(_engine_config(args))
    if args.prompt_ids is not None:
        prompt = [int(t) for t in args.prompt_ids.replace(",", " ").split()]
    elif args.prompt is not None:
        prompt = args.prompt
        if args.chat:  # python/tandem/entrypoints/cli.py:113-114 of 12vivi/tandem
            if engine.tokenizer is None:
                raise SystemExit("--chat needs a tokenizer with a chat template in the model folder")
            prompt = engine.tokenizer.apply_chat_template([{"role": "user", "content": prompt}], tokenize=False,
                                                          add_generation_prompt=True)
    else:
        raise SystemExit("give --prompt (text) or --prompt-ids (token ids)")
    sp = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, top_p=args.top_p,
                        top_k=args.top_k, min_p=args.min_p, seed=args.seed, ignore_eos=args.ignore_eos)
    if args.trace_out:
        engine.record_steps(args.trace_out)
    t0 = time.perf_counter()
    out = engine.generate([prompt], sp)[0]
    dt = time.perf_counter() - t0
    if args.trace_out:
        need = engine.trace.close()
        print(f"[{engine.trace.num_steps} steps written to {args.trace_out}; replay them with "
              f"`tandem replay --model {args.model} --max-tokens {need} --block-size {args.block_size} --out DIR < {args.trace_out}`]",
              file=sys.stderr)
    print(out.text if engine.tokenizer is not None else " ".join(str(t) for t in out.output_token_ids))
    n = len(out.output_token_ids)
    print(f"\n[{n} tokens in {dt:.2f}s, {n / dt:.2f} tok/s, ttft {out.metrics.get('ttft', 0):.3f}s, "
          f"finish={out.finish_reason}]", file=sys.stderr)
    print(json.dumps(engine.stats()), file=sys.stderr)


def cmd_replay(args) -> None:
    from tandem_b200.engine.trace import replay

    def echo(text: str) -> None:
        sys.stdout.write(text + "\n")
        sys.stdout.flush()

    replay(args.model, args.dtype, args.out, args.max_tokens, sys.stdin, args.device, args.block_size, echo)


def cmd_random_model(args) -> None:
    from tandem_b200.weights.random_init import write_random_model

    with open(args.config, encoding="utf-8") as f:
        config = json.load(f)
    print(write_random_model(config, args.out, seed=args.seed, dtype=args.dtype))


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(prog="tandem", description="single-GPU Qwen3 inference engine for B200")
    sub = parser.add_subparsers(dest="cmd", required=True)

    p = sub.add_parser("generate", help="one-off generation")
    _engine_args(p)
    p.add_argument("--prompt", default=None, help="text (needs a tokenizer in the model folder)")
    p.add_argument("--prompt-ids", default=None, help="token ids separated by spaces or commas")
    p.add_argument("--chat", action="store_true", help="wrap the prompt with the tokenizer's chat template")
    p.add_argument("--max-tokens", type=int, default=128)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--top-k", type=int, default=-1)
    p.add_argument("--min-p", type=float, default=0.0)
    p.add_argument("--seed", type=int, default=None)
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--trace-out", default=None, help="write the steps this run takes as a trace that `replay` reads")
    p.set_defaults(fn=cmd_generate)

    p = sub.add_parser("replay", help="replay a trace of steps from stdin and write logits")
    p.add_argument("--model", required=True)
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--out", required=True)
    p.add_argument("--max-tokens", type=int, required=True)
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--block-size", type=int, default=16)
    p.set_defaults(fn=cmd_replay)

    p = sub.add_parser("random-model", help="write a model folder with seeded random weights")
    p.add_argument("--config", required=True, help="a config.json")
    p.add_argument("--out", required=True)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.set_defaults(fn=cmd_random_model)

    args = parser.parse_args(argv)
    args.fn(args)


if __name__ == "__main__":
    main()
