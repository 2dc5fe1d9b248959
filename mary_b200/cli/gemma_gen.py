"""``gemma_gen --pile P --prompt "..." [--max-new N] [--device cuda]``: config-free load from a pile and greedy generation
(src/bin/gemma_gen.rs:77-133).  Without a tokenizer in the pile, ``--ids 1,2,3`` feeds token ids and prints ids."""
from __future__ import annotations

import argparse
import sys
import time

import torch

from ..models.gemma4 import GemmaLM


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="gemma_gen")
    ap.add_argument("--pile", required=True)
    ap.add_argument("--prompt")
    ap.add_argument("--ids")
    ap.add_argument("--max-new", type=int, default=64)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    if argv is None:                                  # run as a program: fail loudly on any thread
        from ..utils import fatal
        fatal.arm()
    dtype = torch.bfloat16 if a.device.startswith("cuda") else torch.float32
    t0 = time.time()
    lm = GemmaLM.from_pile(a.pile, device=a.device, dtype=dtype)
    print(f"loaded in {time.time() - t0:.2f} s", file=sys.stderr)
    t0 = time.time()
    if a.ids:
        out = lm.complete_ids([int(x) for x in a.ids.split(",")], a.max_new)
        print(",".join(map(str, out)))
        n = len(out)
    else:
        text = lm.generate(a.prompt or "", a.max_new)
        print(text)
        n = a.max_new
    print(f"{n / (time.time() - t0):.1f} tok/s", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
