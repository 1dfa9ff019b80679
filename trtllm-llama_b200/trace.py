"""Trace replay: feed given token ids through a served model step by step and write the logits asked for.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--max-seqs 4]

Standard input carries one JSON object per line,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}
Every entry brings the next tokens of one request (admitted at its first entry; it may sit a step out); all entries of a
line run as ONE ragged batch through ``InflightSession.step`` — the step function generation uses — on top of the pages
and state slots earlier steps left.  ``want`` lists the places among the entry's tokens whose logits are written, in the
order of the entries, to OUT/<step>.f32 as little-endian fp32 [wanted, vocab]; requests listed under ``end`` give their
pages and slot back after the step.  After every step the line ``done <step>`` is printed.  Nothing is sampled.

--dtype bfloat16 is the serving mode (bf16 storage and tensor-core products, fp32 accumulation, fp32 residual stream,
norms, softmax and recurrence); float32 keeps every tensor and product in fp32.  The kernels are compiled on the first
call in a fresh checkout (``make ragged``)."""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None):
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder the logits files are written to")
    ap.add_argument("--max-tokens", type=int, required=True, help="positions the cache pool holds (whole pages per request)")
    ap.add_argument("--max-seqs", type=int, default=4, help="state slots = most requests live at any time")
    ap.add_argument("--tokens-per-block", type=int, default=64)
    a = ap.parse_args(argv)

    import torch

    from . import _lib, models
    from .inflight import InflightSession
    from .layers import LayerStackModel

    if not torch.cuda.is_available():
        raise SystemExit("trace_run needs a CUDA device (sm_100a); there is no CPU path")
    _lib.load_ragged_library(build=True)
    model = models.load_model(a.model, dtype=a.dtype, device="cuda")
    if not isinstance(model, LayerStackModel):
        raise SystemExit("trace_run replays models that are served in-flight (ragged batches); this folder holds a "
                         "fixed-batch engine")
    # a request's pages are whole: round the budget up as the pool does
    page = a.tokens_per_block
    sess = InflightSession(model, -(-a.max_tokens // page) * page, a.max_seqs, page)
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        entries = [(e["id"], e["tokens"], e.get("want", [])) for e in msg["entries"]]
        logits = sess.step(entries) if entries else None
        if logits is not None:
            data = logits.cpu().numpy().astype("<f4", copy=False).tobytes()
            tmp = os.path.join(a.out, ".%s.part" % msg["step"])
            with open(tmp, "wb") as f:
                f.write(data)
            os.replace(tmp, os.path.join(a.out, "%s.f32" % msg["step"]))
        else:
            torch.cuda.synchronize()
        for seq_id in msg.get("end", []):
            sess.end(seq_id)
        sys.stdout.write("done %s\n" % msg["step"])
        sys.stdout.flush()
    return 0
