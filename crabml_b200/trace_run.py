"""Replays a trace of steps through a model and writes the logits that the trace asks for.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR [--max-tokens N]

Steps arrive on standard input, one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}

Every entry feeds the NEXT tokens of request `id` (a request's first entry opens a sequence slot); `want` lists the places among
these tokens whose logits are written, in the order of the entries, to OUT/<step>.f32 as little-endian float32 [wanted, vocab].
Requests named in `end` give their slot back after the step.  After every step the line `done <step>` is printed.

The runner samples nothing and has no model code of its own: it drives the registered model's step function and its sequence-state
slots, the ones generation uses."""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def main(argv=None):
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the logits are written to")
    ap.add_argument("--max-tokens", type=int, default=0, help="most tokens live requests hold at any time (sizes the cache of a layer that has no window; other state is bounded per sequence)")
    ap.add_argument("--chunk", type=int, default=0, help="longest run of tokens one pass takes (0: the runner's default)")
    a = ap.parse_args(argv)

    from . import models
    from .tensor import CudaTensorDevice
    device = CudaTensorDevice()
    model = models.load_model(a.model, device, dtype=a.dtype, chunk=a.chunk, max_tokens=a.max_tokens)
    if not hasattr(model, "step"):
        print(f"trace_run: architecture {models.architecture_of(a.model)!r} has no multi-sequence step interface", file=sys.stderr)
        return 3
    os.makedirs(a.out, exist_ok=True)
    slots = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        st = json.loads(line)
        rows = []
        for e in st.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slots[rid] = model.open()
            want = list(e.get("want", []))
            if not e["tokens"]:
                continue
            places = sorted(set(int(i) for i in want))               # the step function takes ascending places; the file keeps the entry's order
            lg = model.step(slots[rid], e["tokens"], places)
            if want:
                rows.append(lg[[places.index(int(i)) for i in want]])
        for rid in st.get("end", []):
            if rid in slots:
                model.close_seq(slots.pop(rid))
        if rows:
            np.concatenate(rows, 0).astype("<f4").tofile(os.path.join(a.out, f"{st['step']}.f32"))
        sys.stdout.write(f"done {st['step']}\n")
        sys.stdout.flush()
    model.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
