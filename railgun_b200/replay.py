"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it
drives ``ModelRunner.step``, the function generation uses.  Steps are read
from standard input, one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` receives the
logits at the wanted places, in the order of the entries and of ``want``, as
little-endian 32-bit floats [wanted, vocab].  After every step a line
``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np


def make_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="bfloat16: the kernels serving uses; float32: everything in true 32-bit")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each request rounded up to 64)")
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--max-requests", type=int, default=8, help="requests live at a time")
    ap.add_argument("--device", default="cuda:0")
    return ap


class Replayer:
    """Feeds trace records to a ModelRunner and writes the wanted logits."""

    def __init__(self, runner, out_dir):
        self.runner = runner
        self.out_dir = Path(out_dir)
        self.out_dir.mkdir(parents=True, exist_ok=True)
        self._ids: dict = {}
        self._next_id = 1

    def _id(self, name):
        if name not in self._ids:
            self._ids[name] = self._next_id
            self._next_id += 1
        return self._ids[name]

    def feed(self, rec: dict) -> None:
        from .engine.batch import StepEntry
        step = rec["step"]
        entries = [StepEntry(self._id(e["id"]), list(e["tokens"]), list(e.get("want", [])))
                   for e in rec.get("entries", [])]
        if entries:
            logits = self.runner.step(entries)
            if logits is not None:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                tmp = self.out_dir / f"{step}.f32.tmp"
                arr.tofile(tmp)
                tmp.replace(self.out_dir / f"{step}.f32")
            self.runner.check_device_errors()
        for name in rec.get("end", []):
            rid = self._ids.pop(name, None)
            if rid is not None:
                self.runner.end([rid])


def main(argv=None) -> int:
    args = make_parser().parse_args(argv)
    from .engine.runner import ModelRunner

    runner = ModelRunner(args.model, dtype=args.dtype, device=args.device, page_size=args.block_size,
                         max_tokens=args.max_tokens, max_requests=args.max_requests)
    replayer = Replayer(runner, args.out)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        replayer.feed(rec)
        print(f"done {rec['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
