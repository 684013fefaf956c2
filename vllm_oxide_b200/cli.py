"""Command line with the reference's options (vllm-oxide, crates/vllm-oxide-cli/src/main.rs:8-85):

    vllm-oxide -m <model folder> [prompt] [--temperature T] [--top-k K] [--top-p P] [--max-tokens N]

The prompt is the positional argument, or all of standard input.  The generated text is printed
(token ids when the model folder has no tokenizer).  Added here: --token-ids, --seed, --dtype, the
engine's sizes, and a mode without a model folder:

    vllm-oxide --random-weights --config <config.json> [--seed N] [--init fan_in|0.02] --token-ids "1 2 3"

which builds the model that config.json describes with seeded random weights: the very values that
`write_random_model_folder` stores for the same seed and scheme (drawn by the host's generator tensor by
tensor, then rounded to the engine's dtype and moved to the device), so a run with --random-weights and a
run from the written folder give the same tokens.
"""
from __future__ import annotations

import argparse
import sys


def parse_args(argv=None):
    ap = argparse.ArgumentParser(prog="vllm-oxide", description="Single-GPU (B200) Qwen3 inference engine")
    ap.add_argument("-m", "--model", default=None, help="local model folder (config.json + safetensors)")
    ap.add_argument("--random-weights", action="store_true",
                    help="no model folder: seeded random weights for the model of --config")
    ap.add_argument("--config", default=None, help="config.json (or a folder that holds one) for --random-weights")
    ap.add_argument("--init", choices=["fan_in", "0.02"], default="fan_in",
                    help="random weights: N(0, 1/fan_in) matrices and N(0, 1) embeddings (default), or N(0, 0.02^2) both")
    ap.add_argument("prompt", nargs="?", default=None, help="prompt text; read from stdin when absent")
    ap.add_argument("--temperature", type=float, default=0.0, help="sampling temperature; 0 = greedy (default)")
    ap.add_argument("--top-k", type=int, default=None, help="keep only the k highest-logit tokens")
    ap.add_argument("--top-p", type=float, default=None, help="keep the smallest token set with cumulative prob >= p")
    ap.add_argument("--max-tokens", type=int, default=16, help="maximum tokens to generate (default 16)")
    ap.add_argument("--token-ids", action="store_true", help="the prompt is a comma/space separated list of token ids")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default=None)
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--block-size", type=int, default=256)
    ap.add_argument("--num-kv-blocks", type=int, default=None)
    ap.add_argument("--ignore-eos", action="store_true")
    args = ap.parse_args(argv)
    if args.random_weights:
        if not args.config or args.model:
            ap.error("--random-weights takes --config <config.json> and no --model")
        if not args.token_ids:
            ap.error("--random-weights has no tokenizer: give the prompt as --token-ids")
    elif not args.model:
        ap.error("one of -m/--model <folder> or --random-weights --config <config.json> is required")
    elif args.config:
        ap.error("--config is only read with --random-weights (a model folder brings its own config.json)")
    return args


def main(argv=None) -> int:
    args = parse_args(argv)
    text = args.prompt if args.prompt is not None else sys.stdin.read()
    from .config.engine_options import EngineOptions
    from .engine.llm import LLM
    from .sampling.params import SamplingParams
    prompt = [int(t) for t in text.replace(",", " ").split()] if args.token_ids else text
    options = EngineOptions(max_model_len=args.max_model_len, block_size=args.block_size,
                            num_kv_blocks=args.num_kv_blocks, dtype=args.dtype, seed=args.seed)
    if args.random_weights:
        import json
        import os
        path = os.path.join(args.config, "config.json") if os.path.isdir(args.config) else args.config
        with open(path) as f:
            config = json.load(f)
        llm = LLM.from_config(config, options, seed=args.seed, init_scheme=args.init, draw_on="cpu")
    else:
        llm = LLM(args.model, options)
    params = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                            max_tokens=args.max_tokens, ignore_eos=args.ignore_eos)
    out = llm.generate([prompt], [params])[0]
    if llm.tokenizer is not None and not args.token_ids:
        print(out.text, end="")
    else:
        print(" ".join(str(t) for t in out.token_ids))
    return 0


if __name__ == "__main__":
    sys.exit(main())
