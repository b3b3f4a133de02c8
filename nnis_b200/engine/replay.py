"""Trace replay: feed given token ids through the engine step by step and
write the logits that are asked for.  Nothing is sampled.

It drives ``Engine.step`` - the model, cache and kernels that generation uses -
and has no forward pass of its own.  The nearest things in NNIS replay a
reference's greedy ids through ``prefill``/``decode_one`` and compare logits per
step (crates/nnis-model/examples/compare_tiny_llama.rs:259-289) or teacher-force
a token list (crates/nnis-cli/src/bin/nnis-kvlab-backend.rs:331-369).

Input, one JSON object per line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

Output: ``<out>/<step>.f32`` (little-endian float32 ``[wanted, vocab]``) for
each step that wants something, and a flushed line ``done <step>`` per step.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, List

import numpy as np
import torch

from .engine import Engine, SequenceStep, StepError


def replay(engine: Engine, lines, out_dir: str, report=None) -> int:
    os.makedirs(out_dir, exist_ok=True)
    slots: Dict[str, int] = {}
    steps = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step_id = record["step"]
        batch: List[SequenceStep] = []
        for entry in record.get("entries", []):
            rid = str(entry["id"])
            if rid not in slots:
                slots[rid] = engine.acquire_slot()
            batch.append(SequenceStep(slots[rid], entry["tokens"], entry.get("want", [])))
        if batch:
            logits = engine.step(batch)
            if logits.shape[0] > 0:
                data = logits.cpu().numpy().astype("<f4", copy=False)
                tmp = os.path.join(out_dir, f".{step_id}.f32.tmp")
                data.tofile(tmp)
                os.replace(tmp, os.path.join(out_dir, f"{step_id}.f32"))
            else:
                torch.cuda.current_stream().synchronize()
            engine.check_status()
        for rid in record.get("end", []):
            rid = str(rid)
            if rid not in slots:
                raise StepError(f"step {step_id}: request {rid!r} ends but never started")
            engine.release_slot(slots.pop(rid))
        steps += 1
        if report is not None:
            report(step_id)
    return steps


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (each rounded up to 64)")
    parser.add_argument("--device", default="cuda:0")
    args = parser.parse_args(argv)
    if args.max_tokens <= 0:
        parser.error("--max-tokens must be positive")
    engine = Engine.from_dir(args.model, dtype=args.dtype, device=args.device,
                             max_tokens=args.max_tokens)

    def report(step_id):
        sys.stdout.write(f"done {step_id}\n")
        sys.stdout.flush()

    replay(engine, sys.stdin, args.out, report)
    return 0
