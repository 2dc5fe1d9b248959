"""``gemma_train_lora --pile P --steps N [--rank 16 --alpha 32 --lr 1e-4 --seq 4096] [--out adapter.safetensors]``.

LoRA finetune of a Gemma-4 decoder loaded from a pile (src/bin/gemma_train_lora.rs:167-335).  Data: ``--ids-file`` with one
comma-separated token sequence per line, or synthetic uniform-random ids.  Under ``torch.distributed.run`` the ranks form a
data-parallel group whose adapter gradients are reduced per layer while backward is still running.  The adapter (and the
optimizer state, for ``--resume``) is committed to the pile; ``--out`` also writes PEFT-named safetensors."""
from __future__ import annotations

import argparse
import sys

import numpy as np
import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="gemma_train_lora")
    ap.add_argument("--pile", required=True)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--rank", type=int, default=16)
    ap.add_argument("--alpha", type=float, default=32.0)
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--ids-file")
    ap.add_argument("--out")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    if argv is None:                                  # run as a program: fail loudly on any thread
        from ..utils import fatal
        fatal.arm()
    from ..format.persist import default_key, load_config, publish_fragment, read_model_pile
    from ..format.selection import SelectedModelIndex
    from ..models.gemma4 import Gemma4Model, Gemma4TextConfig
    from ..models.gemma4.weights import load_into
    from ..nn.weight_loader import WeightLoader
    from ..parallel.group import init_distributed
    from ..pile import Pile, TribleBuilder
    from ..train.trainer import LoraTrainer
    rank, world, local = init_distributed()
    dev = torch.device(a.device if not a.device.startswith("cuda") else f"cuda:{local}")
    pile = Pile.open(a.pile, create=False)
    facts = read_model_pile(pile)
    index = SelectedModelIndex.from_snapshot(pile, facts)
    cfg = Gemma4TextConfig.from_json(load_config(pile, facts, index.roots[0]))
    model = Gemma4Model(cfg, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32, device=dev)
    load_into(model, WeightLoader.from_pile(index))
    reduce_fn = None
    if world > 1:
        import torch.distributed as dist
        reduce_fn = lambda g: dist.all_reduce(g)  # noqa: E731
    tr = LoraTrainer(model, a.rank, a.alpha, a.lr, dp_size=world, reduce_fn=reduce_fn)
    rng = np.random.default_rng(rank)
    if a.ids_file:
        data = [np.array([int(x) for x in line.split(",")], dtype=np.int64) for line in open(a.ids_file) if line.strip()]
    first = last = None
    for step in range(a.steps):
        ids = data[(step * world + rank) % len(data)][:a.seq] if a.ids_file else rng.integers(0, cfg.vocab_size, a.seq)
        loss = tr.step(torch.as_tensor(ids, device=dev)[None])
        first = loss if first is None else first
        last = loss
        if rank == 0:
            print(f"step {step} loss {loss:.4f}")
    if rank == 0:
        tb = TribleBuilder()
        tr.save_checkpoint(pile, tb, index.roots[0])
        publish_fragment(pile, default_key(a.pile), tb.build(), "lora checkpoint")
        if a.out:
            tr.lora.save_safetensors(a.out)
        print(f"first loss {first:.4f} -> last loss {last:.4f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
