"""Trace replay: feed given token ids through a model step by step and write the logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries`` gives every request of the step its next tokens and the places among
them whose logits are wanted; ``end`` names requests that are finished after the
step (their slot and pages are given back).  For a step with wanted places the
logits are written to ``OUT/<step>.f32`` as little-endian float32
[wanted, vocab], in the order of the entries and of ``want``.  After every step
a line ``done <step>`` is printed and flushed.

Nothing is sampled here.  The program drives the same model, step function,
cache and kernels that generation uses and has none of its own.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def run(model_dir: str, dtype: str, out_dir: str, max_tokens: int, lines=None, out=None, device: str = "cuda:0",
        model=None) -> int:
    from .cache import PAGE_SIZE
    from .engine import Engine, Entry, Model

    lines = sys.stdin if lines is None else lines
    out = sys.stdout if out is None else out
    os.makedirs(out_dir, exist_ok=True)
    if model is None:
        model = Model.from_dir(model_dir, dtype=dtype, device=device)
    # every live request holds at least 64 tokens of the budget, so this many can be live at once
    max_seqs = max(1, min(max_tokens // 64, 4096))
    engine = Engine(model, max_tokens=max(max_tokens, PAGE_SIZE), max_seqs=max_seqs)
    slots = {}
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = str(e["id"])
            if rid not in slots:
                slots[rid] = engine.new_sequence()
            entries.append(Entry(slots[rid], e["tokens"], list(e.get("want", []))))
        if entries:
            logits = engine.step(entries)
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(out_dir, f"{step}.f32"))
            elif engine.device.type == "cuda":
                import torch
                torch.cuda.synchronize(engine.device)
            engine.check_device_errors()
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slots:
                engine.release(slots.pop(rid))
        print(f"done {step}", file=out, flush=True)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    a = ap.parse_args(argv)
    return run(a.model, a.dtype, a.out, a.max_tokens)


if __name__ == "__main__":
    sys.exit(main())
