"""Replays a token trace through the engine and writes the logits of the asked positions. Nothing is sampled.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}

Every request id owns a sequence slot of the engine (uzu_engine_slot_acquire) from its first step until a step lists it under "end";
a step feeds each entry's next tokens to its slot (uzu_engine_forward_rows: the engine's pass driver, caches, recurrent states and
kernels) and the f32 logits of the "want" indices go to DIR/<step>.f32, [wanted, vocab] little-endian, in the order of the entries.
After every step the line `done <step>` is printed. The library is compiled on first use when the checkout has none.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import numpy as np


def ensure_library():
    """Build libuzu_b200.so in the checkout when it is missing or stale; one builder at a time (other processes wait on the lock)."""
    import fcntl

    from . import build as ubuild
    ubuild.OBJ.mkdir(exist_ok=True)
    with open(ubuild.OBJ / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        ubuild.build()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description="feed given token ids through a model step by step and write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                    help="bfloat16: the serving precisions (bf16 products, f32 accumulation and f32 sums / norms / scores / states); float32: everything in true f32")
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, default=8192, help="most tokens that live requests hold at any time (sizes the caches)")
    ap.add_argument("--device", type=int, default=-1)
    a = ap.parse_args(argv)

    ensure_library()
    from . import binding as B

    out_dir = Path(a.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    ctx = B.Context(a.device)
    eng = B.Engine(ctx, a.model, max_context_length=max(int(a.max_tokens), 16), use_cuda_graph=False, storage_f32=(a.dtype == "float32"))
    slots: dict[str, int] = {}
    try:
        for line in sys.stdin:
            line = line.strip()
            if not line:
                continue
            step = json.loads(line)
            parts = []
            for ent in step.get("entries", []):
                rid = str(ent["id"])
                if rid not in slots:
                    slots[rid] = eng.slot_acquire()
                tokens = ent.get("tokens", [])
                want = sorted(ent.get("want", []))
                if want != list(ent.get("want", [])):
                    raise ValueError("'want' must be ascending")
                if tokens:
                    logits = eng.forward_rows(tokens, want, slot=slots[rid])
                    if len(want):
                        parts.append(logits)
            for rid in step.get("end", []):
                rid = str(rid)
                if rid in slots:
                    eng.slot_release(slots.pop(rid))
            if parts:
                tmp = out_dir / f".{step['step']}.f32.tmp"
                np.concatenate(parts, axis=0).astype("<f4").tofile(tmp)
                os.replace(tmp, out_dir / f"{step['step']}.f32")
            sys.stdout.write(f"done {step['step']}\n")
            sys.stdout.flush()
    finally:
        eng.close()
        ctx.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
