"""Command line: MODEL_DIR [PROMPT_IDS] [MAX_NEW_TOKENS], after the reference's
`llama_generate MODEL_DIR ["PROMPT"] [MAX_NEW_TOKENS]` (examples/llama_generate.rs:68-81): the
same positional arguments, the same default of 32 new tokens, generation defaults from the
folder's generation_config.json, one batched prefill and cached one-token steps.  This library has
no tokenizer, so the prompt is token ids: "464,1115,4165"; several prompts are separated by ";".
Options carry the names of the reference's GenerationConfig fields."""
from __future__ import annotations

import argparse
import json
import sys

USAGE = "usage: generate MODEL_DIR [PROMPT_IDS] [MAX_NEW_TOKENS] [options]"


def parse_prompts(text: str) -> list[list[int]]:
    prompts = []
    for part in text.split(";"):
        ids = [int(x) for x in part.replace(",", " ").split()]
        if not ids:
            raise ValueError("an empty prompt")
        prompts.append(ids)
    return prompts


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="generate", description=__doc__, usage=USAGE,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("model_dir")
    parser.add_argument("prompt_ids", nargs="?", default="464,1115,4165,7577,389")
    parser.add_argument("max_new_tokens", nargs="?", type=int, default=32)
    parser.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    parser.add_argument("--strategy", choices=["greedy", "sample"], default=None)
    parser.add_argument("--temperature", type=float, default=None)
    parser.add_argument("--top-k", type=int, default=None)
    parser.add_argument("--top-p", type=float, default=None)
    parser.add_argument("--min-p", type=float, default=None)
    parser.add_argument("--repetition-penalty", type=float, default=None)
    parser.add_argument("--presence-penalty", type=float, default=None)
    parser.add_argument("--frequency-penalty", type=float, default=None)
    parser.add_argument("--no-repeat-ngram-size", type=int, default=None)
    parser.add_argument("--min-new-tokens", type=int, default=None)
    parser.add_argument("--seed", type=int, default=None)
    parser.add_argument("--eos-token-ids", type=str, default=None, help="comma-separated ids")
    parser.add_argument("--stop-sequences", type=str, default=None, help='"1,2;3" = two stop sequences')
    parser.add_argument("--max-batch", type=int, default=None)
    parser.add_argument("--prefill-chunk-size", type=int, default=None,
                        help="the most tokens of a prompt one step brings (default: whole prompts in one step)")
    parser.add_argument("--json", action="store_true", help="print one JSON object per sequence")
    args = parser.parse_args(argv)
    if args.max_new_tokens <= 0:
        print(USAGE, file=sys.stderr)
        return 2

    from .auto import AutoCausalLm, AutoLoadOptions, CausalGenerationRequest, cache_tokens_for, generate_causal
    from .errors import BurnTransformersError

    try:
        prompts = parse_prompts(args.prompt_ids)
    except ValueError as error:
        print(f"generate: cannot read PROMPT_IDS: {error}\n{USAGE}", file=sys.stderr)
        return 2
    try:
        tokens = cache_tokens_for([len(p) for p in prompts], args.max_new_tokens)
        loaded = AutoCausalLm.load_local(args.model_dir, AutoLoadOptions(dtype=args.dtype, max_tokens=tokens))
        generation = loaded.generation_defaults
        generation.max_new_tokens = args.max_new_tokens
        for name in ("strategy", "temperature", "top_k", "top_p", "min_p", "repetition_penalty", "presence_penalty",
                     "frequency_penalty", "no_repeat_ngram_size", "min_new_tokens", "seed"):
            value = getattr(args, name)
            if value is not None:
                setattr(generation, name, value)
        if args.temperature is not None and args.strategy is None:
            generation.strategy = "sample"
        if args.eos_token_ids is not None:
            generation.eos_token_ids = [int(x) for x in args.eos_token_ids.split(",") if x.strip()]
        if args.stop_sequences is not None:
            generation.stop_sequences = parse_prompts(args.stop_sequences)
        output = generate_causal(loaded.model, CausalGenerationRequest(prompts, generation, args.max_batch,
                                                                      args.prefill_chunk_size))
    except BurnTransformersError as error:
        print(f"generate: {error}", file=sys.stderr)
        return 1
    for prompt, sequence in zip(prompts, output.sequences):
        if args.json:
            print(json.dumps({"prompt": prompt, "token_ids": sequence.token_ids,
                              "log_probabilities": sequence.log_probabilities,
                              "finish_reason": dataclass_dict(sequence.finish_reason)}))
        else:
            print(" ".join(str(t) for t in prompt + sequence.token_ids))
    return 0


def dataclass_dict(reason):
    return {k: v for k, v in vars(reason).items() if v is not None} if reason else None


if __name__ == "__main__":
    sys.exit(main())
