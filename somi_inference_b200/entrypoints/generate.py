"""Command line: generate tokens from a model folder, or write a random model folder.

    python -m somi_inference_b200.entrypoints.generate --model-name DIR --prompt-ids 5 17 3 \\
        --max-new-tokens 16 --temperature 0
    python -m somi_inference_b200.entrypoints.generate --config CONFIG.json --random-weights --seed 0 \
        --prompt-lens 5 17 33 --max-new-tokens 8 --temperature 0
    python -m somi_inference_b200.entrypoints.generate --write-random-model DIR --config CONFIG.json --seed 0

The second form goes from a configuration and a seed to tokens in one call: the weights are drawn
as `--write-random-model` would write them and handed to the engine in memory.

The reference ships no command line of its own inside the package; its programs
are the `python -m benchmarks.bench_*` scripts, whose option names are kept
where they mean the same thing: `--model-name`, `--block-size`, `--device`,
`--dtype`, `--seed`, `--prompt-lens` (benchmarks/bench_decode.py:116-199,
benchmarks/bench_prefill.py:44-118).  The `LLM` options keep their names too:
`--num-blocks`, `--max-concurrent` (somi_inference/entrypoints/llm.py:58-70) and
the sampling options of `generate` (llm.py:126-135).
"""

from __future__ import annotations

import argparse
import json
import sys

import torch


def parse_args(argv: list[str] | None = None) -> argparse.Namespace:
    p = argparse.ArgumentParser(prog="somi_inference_b200.entrypoints.generate",
                                description="Generate with the B200 engine.")
    p.add_argument("--model-name", type=str, help="Model folder (config.json + safetensors).")
    p.add_argument("--block-size", type=int, default=16, help="KV cache block size.")
    p.add_argument("--num-blocks", type=int, default=256, help="KV cache blocks per layer group.")
    p.add_argument("--max-concurrent", type=int, default=16, help="Most requests running at once.")
    p.add_argument("--device", type=str, default="auto", choices=["auto", "cuda"],
                   help="Execution device; the engine has no CPU path.")
    p.add_argument("--dtype", type=str, default="auto",
                   choices=["auto", "float32", "bfloat16"],
                   help="Model / cache dtype. 'auto' is bfloat16.")
    p.add_argument("--seed", type=int, default=42,
                   help="Random seed for prompt generation, synthetic weights and sampling.")
    p.add_argument("--prompt", type=str, default=None, help="Text prompt (needs tokenizer files).")
    p.add_argument("--prompt-ids", type=int, nargs="+", default=None, help="Prompt as token ids.")
    p.add_argument("--prompt-lens", type=int, nargs="+", default=None,
                   help="Random prompts of these lengths, run together.")
    p.add_argument("--max-new-tokens", type=int, default=16)
    p.add_argument("--temperature", type=float, default=1.0)
    p.add_argument("--top-k", type=int, default=-1)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--repetition-penalty", type=float, default=1.0)
    p.add_argument("--chunk-size", type=int, default=512, help="Largest prompt portion per step.")
    p.add_argument("--max-num-batched-tokens", type=int, default=2048)
    p.add_argument("--policy", choices=["preempt", "reserve"], default="preempt")
    p.add_argument("--write-random-model", type=str, default=None, metavar="DIR",
                   help="Write config.json + model.safetensors with random weights and exit.")
    p.add_argument("--config", type=str, default=None,
                   help="config.json to take the sizes from (with --write-random-model or "
                        "--random-weights).")
    p.add_argument("--random-weights", action="store_true",
                   help="Generate with random weights drawn from --seed for the model of --config "
                        "(no model folder needed).")
    p.add_argument("--std", type=float, default=0.02,
                   help="Standard deviation of the random weights.")
    p.add_argument("--weights-dtype", choices=["float32", "bfloat16"], default="bfloat16")
    p.add_argument("--output-file", type=str, default=None, help="Append results as JSONL.")
    return p.parse_args(argv)


def _typed_config(path: str):
    from ..config.registry import config_class_for
    with open(path) as f:
        raw = json.load(f)
    archs = raw.get("architectures")
    if not archs:
        raise ValueError(f"{path}: no 'architectures' list")
    return config_class_for(archs[0]).from_dict(raw)


def main(argv: list[str] | None = None, *, ops=None, device=None) -> int:
    """`ops` and `device` are for tests that run the command line without a GPU."""
    args = parse_args(argv)
    if args.write_random_model:
        if not args.config:
            print("--write-random-model needs --config", file=sys.stderr)
            return 2
        from ..weights import write_random_model
        write_random_model(_typed_config(args.config), args.seed, args.write_random_model,
                           dtype=getattr(torch, args.weights_dtype), std=args.std)
        print(args.write_random_model)
        return 0
    if args.random_weights and not args.config:
        print("--random-weights needs --config", file=sys.stderr)
        return 2
    if not args.model_name and not args.random_weights:
        print("--model-name (or --config with --random-weights) is required", file=sys.stderr)
        return 2
    if args.prompt is None and args.prompt_ids is None and args.prompt_lens is None:
        print("give --prompt, --prompt-ids or --prompt-lens", file=sys.stderr)
        return 2
    from ..engine import LLM, Engine
    from ..sampling import SamplingParams
    dtype = "bfloat16" if args.dtype == "auto" else args.dtype
    common = dict(max_concurrent=args.max_concurrent, chunk_size=args.chunk_size,
                  max_num_batched_tokens=args.max_num_batched_tokens, policy=args.policy)
    if args.random_weights:
        from ..weights import random_tensors
        cfg = _typed_config(args.config)
        tensors = random_tensors(cfg, args.seed, std=args.std,
                                 dtype=getattr(torch, args.weights_dtype))
        engine = Engine.from_tensors(cfg, tensors, dtype=dtype, page_size=args.block_size,
                                     num_pages=args.num_blocks, max_requests=args.max_concurrent,
                                     **({"ops": ops} if ops is not None else {}),
                                     **({"device": device} if device is not None else {}))
        llm = LLM(engine, **common)
    else:
        llm = LLM(args.model_name, num_blocks=args.num_blocks, block_size=args.block_size,
                  dtype=dtype, ops=ops, device=device, **common)
    kw = dict(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
              repetition_penalty=args.repetition_penalty)
    results = []
    if args.prompt is not None:
        text = llm.generate(args.prompt, max_new_tokens=args.max_new_tokens, seed=args.seed, **kw)
        results.append({"prompt": args.prompt, "text": text})
    elif args.prompt_ids is not None:
        out = llm.generate(args.prompt_ids, max_new_tokens=args.max_new_tokens, seed=args.seed, **kw)
        results.append({"prompt_ids": args.prompt_ids, "output_ids": out})
    elif args.prompt_lens is not None:
        g = torch.Generator().manual_seed(args.seed)
        prompts = [torch.randint(0, llm.config.vocab_size, (n,), generator=g).tolist()
                   for n in args.prompt_lens]
        sps = [SamplingParams(seed=args.seed + i, **kw) for i in range(len(prompts))]
        outs = llm.generate_many(prompts, max_new_tokens=args.max_new_tokens, sampling_params=sps,
                                 ignore_eos=True)
        results = [{"prompt_len": n, "output_ids": o} for n, o in zip(args.prompt_lens, outs)]
    for r in results:
        print(json.dumps(r))
    if args.output_file:
        with open(args.output_file, "a") as f:
            for r in results:
                f.write(json.dumps(r) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
