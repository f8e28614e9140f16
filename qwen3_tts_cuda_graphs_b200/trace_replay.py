"""Replay a token trace through a sequence model, step by step, and write the logits of the asked positions.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N   < steps.jsonl

Every input line is one step: {"step": n, "entries": [{"id": ..., "tokens": [...], "want": [...]}], "end": [...]}.  Each entry's
tokens go through `SequenceEngine.step` (the generation path's step function: same op lists, state slots and kernels) from the
state the request's earlier steps left; the logits at the `want` positions, in entry order, are written to DIR/<n>.f32
(little-endian f32 [wanted, vocab]) and "done <n>" is printed.  Requests named in "end" give their slot back.  Nothing is sampled.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, help="directory with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    ap.add_argument("--out", required=True, help="directory for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, default=4096, help="most tokens live requests hold at any time")
    ap.add_argument("--max-slots", type=int, default=4, help="most requests alive at once")
    a = ap.parse_args(argv)

    import torch

    from .seq_engine import SequenceEngine

    if not torch.cuda.is_available():
        print("trace_run needs a CUDA device (there is no CPU fallback)", file=sys.stderr)
        return 2
    os.makedirs(a.out, exist_ok=True)
    eng = SequenceEngine.from_pretrained(a.model, "cuda", a.dtype, max_tokens=max(1, a.max_tokens), max_slots=max(1, a.max_slots))
    out = sys.stdout
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        st = json.loads(line)
        rows = []
        for e in st.get("entries", []):
            lg = eng.step(e["id"], e["tokens"], e.get("want") or [])
            if lg is not None:
                rows.append(lg.to("cpu", copy=True))
        for r in st.get("end", []):
            eng.close(r)
        if rows:
            data = torch.cat(rows, 0).to(torch.float32).contiguous().numpy()
            if sys.byteorder != "little":
                data = data.byteswap()
            tmp = os.path.join(a.out, ".%d.part" % st["step"])
            with open(tmp, "wb") as f:
                f.write(data.tobytes())
            os.replace(tmp, os.path.join(a.out, "%d.f32" % st["step"]))
        else:
            torch.cuda.synchronize()
        out.write("done %d\n" % st["step"])
        out.flush()
    eng.close_all()
    return 0


if __name__ == "__main__":
    sys.exit(main())
