"""Command line: generate tokens from a model folder, or write a random model folder.

    python -m somi_inference_b200.entrypoints.generate --model-name DIR --prompt-ids 5 17 3 \\
        --max-new-tokens 16 --temperature 0
    python -m somi_inference_b200.entrypoints.generate --write-random-model DIR --config CONFIG.json --seed 0

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
                   help="config.json to take the sizes from (with --write-random-model).")
    p.add_argument("--weights-dtype", choices=["float32", "bfloat16"], default="bfloat16")
    p.add_argument("--output-file", type=str, default=None, help="Append results as JSONL.")
    return p.parse_args(argv)


def main(argv: list[str] | None = None) -> int:
    args = parse_args(argv)
    if args.write_random_model:
        if not args.config:
            print("--write-random-model needs --config", file=sys.stderr)
            return 2
        from ..config.registry import config_class_for
        from ..weights import write_random_model
        with open(args.config) as f:
            raw = json.load(f)
        cfg = config_class_for(raw["architectures"][0]).from_dict(raw)
        write_random_model(cfg, args.seed, args.write_random_model,
                           dtype=getattr(torch, args.weights_dtype))
        print(args.write_random_model)
        return 0
    if not args.model_name:
        print("--model-name is required", file=sys.stderr)
        return 2
    from ..engine import LLM
    from ..sampling import SamplingParams
    dtype = "bfloat16" if args.dtype == "auto" else args.dtype
    llm = LLM(args.model_name, num_blocks=args.num_blocks, block_size=args.block_size,
              max_concurrent=args.max_concurrent, dtype=dtype, chunk_size=args.chunk_size,
              max_num_batched_tokens=args.max_num_batched_tokens, policy=args.policy)
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
    else:
        print("give --prompt, --prompt-ids or --prompt-lens", file=sys.stderr)
        return 2
    for r in results:
        print(json.dumps(r))
    if args.output_file:
        with open(args.output_file, "a") as f:
            for r in results:
                f.write(json.dumps(r) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
