"""Trace replay over the engine's own step function (see ``bin/trace_run``)."""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, List

import numpy as np


def main(argv: List[str]) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description="replay token traces and write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", required=True, type=int,
                    help="most tokens that live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    import torch
    from .engine import Engine, Model

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; quicknn_b200 has no CPU path", file=sys.stderr)
        return 3
    os.makedirs(args.out, exist_ok=True)
    model = Model.from_folder(args.model, args.dtype, args.device)
    engine = Engine(model, max_tokens=args.max_tokens)
    slots: Dict[str, int] = {}

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step_id = rec["step"]
        entries, want = [], []
        for e in rec.get("entries", []):
            rid = str(e["id"])
            if rid not in slots:
                slots[rid] = engine.new_sequence()
            entries.append((slots[rid], [int(t) for t in e["tokens"]]))
            want.append([int(i) for i in e.get("want", [])])
        if entries:
            logits = engine.step(entries, want)
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(args.out, f"{step_id}.f32"))
            else:
                torch.cuda.synchronize()
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slots:
                engine.release(slots.pop(rid))
        print(f"done {step_id}", flush=True)
    return 0
