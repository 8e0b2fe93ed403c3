#!/usr/bin/env python3
"""Replay a trace of token ids through a checkpoint and write the logits — nothing is sampled.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps arrive on standard input, one JSON object per line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}

All entries of a step form one batch and run from the state earlier steps left; ``want`` lists the places among an
entry's tokens whose logits are written to ``<out>/<step>.f32`` (little-endian fp32 ``[wanted, vocab]``, entry
order); ``end`` names the requests whose slots are given back afterwards.  After every step ``done <step>`` is
printed.  The model class comes from the checkpoint's ``config.json`` through the model registry, and the step runs
through the same runner, state pool and kernels as generation (``parallel/hybrid_runner.py``).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="Replay a token trace and write logits")
    p.add_argument("--model", type=Path, required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--out", type=Path, required=True)
    p.add_argument("--max-tokens", type=int, default=4096, help="most tokens live requests hold at any time")
    p.add_argument("--device", default=None)
    return p


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    import torch

    from ..models.hybrid import load_hybrid
    from ..models.registry import architecture_of
    from ..parallel.hybrid_runner import HybridRunner

    if not architecture_of(args.model):
        print(f"{args.model}: no config.json with an 'architecture' entry", file=sys.stderr)
        return 2
    device = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    dtype = getattr(torch, args.dtype)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    model = load_hybrid(args.model, device, dtype)
    runner = HybridRunner(model, max_seq_length=max(1, args.max_tokens))
    args.out.mkdir(parents=True, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = [(e["id"], e["tokens"]) for e in step.get("entries", [])]
        want = [e.get("want", []) for e in step.get("entries", [])]
        if entries:
            logits = runner.step(entries, want)
            if logits.size(0):
                (args.out / f"{step['step']}.f32").write_bytes(logits.float().cpu().contiguous().numpy().astype("<f4").tobytes())
        for rid in step.get("end", []):
            if rid in runner.slots:
                runner.end_sample(rid)
        print(f"done {step['step']}", flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
