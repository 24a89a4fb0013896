"""Command line in the manner of the reference's `rustml-infer`
(`rustml/nlp/main/src/bin/infer.rs:14-49`): the same option names and meanings where it has
them (`--prompt`, `--max-tokens` default 256, `--temperature` default 0.8 with 0.0 = greedy,
`--top-k`, `--top-p`, `--repetition-penalty`, `--stream`), a model folder instead of a GGUF file
(or `--random-config FILE.json --weights-seed N`: random weights made on the device from a
configuration), and token ids instead of text: `--prompt-ids` and `--prompt-file` (one sequence of ids a line; the
lines run together as one batch).  `--prompt TEXT` is kept for demonstrations and maps the text's
UTF-8 bytes to ids, as the reference's byte tokenizer does (`rustml/tokenizer/main/src/core/byte.rs:7`).
`--chat` is not carried over: templates are the tokenizer's side.  Diagnostics go to standard
error, generated ids to standard output (`infer.rs:71-119, 145-158`); among them the model's
sizes (`infer.rs:86-89`) and, after the run, prompt and decode rates in the wording of
`rustml/nlp/examples/gemma3_gguf.rs:43-46, :73`.  `--timings` adds the device time of every step.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import List, Optional


def _parse_ids(text: str) -> List[int]:
    try:
        return [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise SystemExit(f"error: token ids must be integers, got {text!r}") from None


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="rustml-infer", description="Generate with a model folder (config.json + "
                                "model.safetensors) on one B200.")
    p.add_argument("model_dir", metavar="MODEL_DIR", nargs="?", default=None,
                   help="Path to a model folder (or give --random-config).")
    p.add_argument("--random-config", metavar="JSON", default=None,
                   help="config.json of a model to build with random weights N(0, 0.02) instead of loading MODEL_DIR.")
    p.add_argument("--weights-seed", type=int, default=None, help="Seed of the random weights (default: --seed).")
    p.add_argument("--prompt", help="Prompt text (its UTF-8 bytes become token ids). Reads from stdin if no prompt option is given.")
    p.add_argument("--prompt-ids", help="Prompt as token ids, separated by commas or spaces.")
    p.add_argument("--prompt-file", help="File with one prompt a line, as token ids; the lines are generated as a batch.")
    p.add_argument("--max-tokens", type=int, default=256, help="Maximum number of tokens to generate.")
    p.add_argument("--temperature", type=float, default=0.8, help="Sampling temperature (0.0 = greedy).")
    p.add_argument("--top-k", type=int, default=None, help="Top-k sampling.")
    p.add_argument("--top-p", type=float, default=None, help="Nucleus (top-p) sampling.")
    p.add_argument("--repetition-penalty", type=float, default=None, help="Repetition penalty.")
    p.add_argument("--stream", action="store_true", help="Print tokens as they are generated.")
    p.add_argument("--seed", type=int, default=0, help="Seed of the sampler.")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                   help="bfloat16: the serving kernels; float32: everything in true 32-bit.")
    p.add_argument("--stop-ids", default=None, help="Stop token ids (default: the model's end-of-sequence ids).")
    p.add_argument("--max-context", type=int, default=None, help="Longest sequence the cache is sized for.")
    p.add_argument("--timings", action="store_true", help="Print the device time of every step (CUDA events) to stderr.")
    return p


def read_prompts(args, stdin) -> List[List[int]]:
    given = [a for a in (args.prompt, args.prompt_ids, args.prompt_file) if a is not None]
    if len(given) > 1:
        raise SystemExit("error: give one of --prompt, --prompt-ids, --prompt-file")
    if args.prompt_ids is not None:
        prompts = [_parse_ids(args.prompt_ids)]
    elif args.prompt_file is not None:
        try:
            with open(args.prompt_file) as f:
                prompts = [_parse_ids(line) for line in f if line.strip()]
        except OSError as e:
            raise SystemExit(f"error: cannot read {args.prompt_file}: {e.strerror}") from None
    else:
        text = args.prompt
        if text is None:
            print("Reading prompt from stdin...", file=sys.stderr)
            text = stdin.read()
        if not text.strip():
            # the reference's message, infer.rs:60-62
            raise SystemExit("error: No prompt provided (use --prompt or pipe text to stdin)")
        prompts = [list(text.encode("utf-8"))]
    if not prompts or any(len(p) == 0 for p in prompts):
        raise SystemExit("error: an empty prompt")
    return prompts


def main(argv: Optional[List[str]] = None, stdin=None, stdout=None) -> int:
    args = build_parser().parse_args(argv)
    stdin, stdout = stdin or sys.stdin, stdout or sys.stdout
    if (args.model_dir is None) == (args.random_config is None):
        raise SystemExit("error: give either MODEL_DIR or --random-config FILE.json")
    prompts = read_prompts(args, stdin)

    from .config.base import ConfigError
    from .engine.api import Generator, load_model, random_model
    from .engine.generate import GenerationStats
    from .weights.loader import WeightError
    from .weights.safetensors_io import SafetensorsError

    try:
        if args.random_config is not None:
            weights_seed = args.seed if args.weights_seed is None else args.weights_seed
            print(f"Building random weights from {args.random_config} (seed {weights_seed}, {args.dtype})...", file=sys.stderr)
            try:
                with open(args.random_config) as f:
                    raw = json.load(f)
            except (OSError, ValueError) as e:
                print(f"error: cannot read {args.random_config}: {e}", file=sys.stderr)
                return 1
            model = random_model(raw, weights_seed, args.dtype)
        else:
            print(f"Loading {args.model_dir} ({args.dtype})...", file=sys.stderr)
            model = load_model(args.model_dir, args.dtype)
    except (ConfigError, WeightError, SafetensorsError, RuntimeError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    spec = model.spec
    print(f"  arch={spec.architecture}, dim={spec.hidden_size}, layers={len(spec.layers)}, vocab={spec.vocab_size}",
          file=sys.stderr)
    from .cache.cache import CacheError
    from .engine.step import StepError

    def on_token(request, token):
        stdout.write(f"{request}\t{token}\n" if len(prompts) > 1 else f"{token}\n")
        stdout.flush()

    stats = GenerationStats()
    try:
        # what the user's numbers can get wrong (a context shorter than a prompt, an id outside the vocabulary, a
        # sampling option outside its range) comes back as the library's own errors: one line, no traceback
        if args.max_context is not None and args.max_context < 1:
            raise ValueError("--max-context must be at least 1")
        longest = max(len(p) for p in prompts) + max(args.max_tokens, 0)
        gen = Generator(model, max_batch=min(len(prompts), 64), max_context=args.max_context or min(longest, model.max_positions),
                        time_steps=args.timings)
        gen.with_temperature(args.temperature).with_top_k(args.top_k).with_top_p(args.top_p)
        gen.with_repetition_penalty(args.repetition_penalty).with_seed(args.seed)
        if args.stop_ids is not None:
            gen.with_stop_tokens(_parse_ids(args.stop_ids))
        print(f"Generating up to {args.max_tokens} tokens for {len(prompts)} prompt(s)...", file=sys.stderr)
        results = gen.generate_batch_results(prompts, args.max_tokens, stream=on_token if args.stream else None, stats=stats)
    except (StepError, CacheError, ValueError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    if not args.stream:
        for r in results:
            stdout.write(" ".join(str(t) for t in r.tokens) + "\n")
    for i, r in enumerate(results):
        print(f"prompt {i}: {len(r.tokens)} tokens, finished by {r.finish_reason}", file=sys.stderr)
    print(f"  Prefill: {stats.prefill_tokens} tokens in {stats.prefill_seconds:.2f}s ({stats.prefill_rate():.1f} tok/s)", file=sys.stderr)
    print(f"  Decode: {stats.decode_tokens} tokens in {stats.decode_seconds:.2f}s ({stats.decode_rate():.1f} tok/s)", file=sys.stderr)
    if args.timings:
        for k, t in enumerate(gen.engine.step_timings()):
            print(f"  step {k}: {t['kind']}, {t['sequences']} sequences, {t['tokens']} tokens, {t['ms']:.3f} ms", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
