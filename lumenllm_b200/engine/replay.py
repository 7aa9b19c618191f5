"""Trace replay: feeds given token ids through a model step by step and writes
logits. It samples nothing and has no forward pass, cache or loader of its own:
it drives the Engine that generation uses.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, DIR/<step>.f32 receives the logits at
the wanted places as little-endian float32 [wanted, vocab], in the order of the
entries and of `want`. After every step a line `done <step>` is printed and
flushed. Requests named in `end` give back what they hold after the step.

The reference's seeds for this tool are `forward_logits` per token
(crates/aegisllm-base/src/executor/traits.rs:73-74) and its chunk-sweep check
(crates/aegisllm/src/cli/smoke.rs:109-131).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    args = ap.parse_args(argv)

    from .engine import Engine, StepEntry
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    engine = Engine.from_folder(args.model, dtype=args.dtype, max_tokens=args.max_tokens)
    slots = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slots[rid] = engine.alloc_slot()
            entries.append(StepEntry(slots[rid], e["tokens"], e.get("want", ())))
        if entries:
            logits = engine.step(entries)
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu").contiguous().numpy().astype("<f4", copy=False)
                engine.check_kernels()         # logits of a kernel that gave up are not written
                arr.tofile(out / f"{step}.f32")
        for rid in rec.get("end", []):
            if rid in slots:
                engine.free_slot(slots.pop(rid))
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
