"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives the
library's model, step function, cache and kernels, the ones generation uses.  (The
reference's nearest tools are `rustml/experimentation/llmforge/examples/logit_dump.rs:125-254`,
prefill plus three greedy steps with top-20 logits, and the printed comparison in
`rustml/nlp/tests/forward_diagnostic_test.rs:61-150`.)

Input: one JSON object per line on standard input,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries` gives each request's next tokens and the places among them whose logits are wanted;
`end` names requests that are finished after the step (their slot and pages are given back).
For a step that wants something, `<out>/<step>.f32` receives the logits at the wanted places,
in the order of the entries and of `want`, as little-endian float32 [wanted, vocab].
After every step a line `done <step>` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys



def run(argv=None, stdin=None, stdout=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"],
                    help="bfloat16: the serving kernels; float32: everything in true 32-bit")
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to a multiple of the page size (64)")
    args = ap.parse_args(argv)
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout

    from ..cache.cache import DEFAULT_PAGE_SIZE, CacheError
    from ..config.base import ConfigError
    from ..weights.loader import WeightError
    from ..weights.safetensors_io import SafetensorsError
    from .api import load_model
    from .step import Engine, StepError

    os.makedirs(args.out, exist_ok=True)
    try:
        model = load_model(args.model, args.dtype)
    except (ConfigError, WeightError, SafetensorsError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    page = DEFAULT_PAGE_SIZE     # the unit requests' token counts are rounded up to
    max_tokens = max(page, -(-args.max_tokens // page) * page)
    engine = Engine(model, max_tokens=max_tokens, max_seqs=max_tokens // page,
                    max_context=min(model.max_positions, max_tokens), page_size=page)
    slots = {}
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        step = None
        try:
            msg = json.loads(line)
            step = msg["step"]
            entries = msg.get("entries", [])
            if entries:
                ids = [e["id"] for e in entries]
                for rid in ids:
                    if rid not in slots:
                        slots[rid] = engine.new_sequence()
                want = [list(e.get("want", [])) for e in entries]
                logits = engine.step([slots[r] for r in ids], [e["tokens"] for e in entries], want)
                if sum(len(w) for w in want):
                    data = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                    engine.check_status()
                    tmp = os.path.join(args.out, f"{step}.f32.tmp")
                    data.tofile(tmp)
                    os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
            for rid in msg.get("end", []):
                if rid in slots:
                    engine.release(slots.pop(rid))
        except (ValueError, KeyError, TypeError, AttributeError, StepError, CacheError) as e:
            # a line that is no step, or a step the engine refuses (an id outside the vocabulary, more tokens than
            # --max-tokens promised): say which and stop; nothing is written for it
            what = f"{type(e).__name__}: {e}" if not isinstance(e, (StepError, CacheError)) else str(e)
            print(f"error: step {step if step is not None else '?'}: {what}", file=sys.stderr)
            return 1
        stdout.write(f"done {step}\n")
        stdout.flush()
    if engine.device.type == "cuda":
        import torch
        torch.cuda.synchronize()
    engine.check_status()        # also for steps that wanted nothing
    return 0


def main():
    try:
        sys.exit(run())
    except BrokenPipeError:
        sys.exit(1)


if __name__ == "__main__":
    main()
