"""``GemmaLM``: the in-process generation seam (src/models/gemma/gemma4/lm.rs:46-372).

``from_pile`` is config-free: hyper-parameters and tokenizer come from facts in the pile.  ``generate`` applies the
chat template ``<bos><|turn>user\\n...<turn|>\\n<|turn>model\\n`` (:127), decodes greedily (first maximum wins,
:22-32) and stops on id 1, ``<turn|>``, the token budget or a stop string (:172-201); ``complete_ids`` is the
raw id-level entry used by parity tests (:316-371)."""
from __future__ import annotations

import torch

from ...format.persist import load_config, read_model_pile
from ...format.selection import ModelSelector, SelectedModelIndex
from ...nn.weight_loader import WeightLoader
from ...pile import Pile
from ...runtime.engine import Engine
from ...runtime.kv_cache import PagedKVCache
from .config import Gemma4TextConfig
from .model import Gemma4Model
from .weights import load_into

EOS_ID = 1


class GemmaLM:
    def __init__(self, model: Gemma4Model, tokenizer=None, device="cpu", max_seq: int = 4096, page_size: int = 16,
                 max_batch: int = 8):
        self.model, self.tokenizer, self.device = model, tokenizer, torch.device(device)
        spec = model.kv_spec()
        pages = max_batch * ((max_seq + page_size - 1) // page_size) + 8
        self.cache = PagedKVCache(spec["num_layers"], pages, page_size, spec["kv_heads"], spec["head_dim"],
                                  dtype=model.dtype, device=device)
        eos = {EOS_ID}
        if tokenizer is not None:
            t = tokenizer.token_to_id("<turn|>")
            if t is not None:
                eos.add(t)
        self.engine = Engine(model, self.cache, max_tokens=max(2048, max_batch), max_seqs=max_batch,
                             prefill_chunk=2048, device=device, eos_ids=eos)

    @staticmethod
    def from_pile(path, selector: ModelSelector = ModelSelector.only(), device="cpu", dtype=torch.float32, **kw) -> "GemmaLM":
        pile = Pile.open(str(path), create=False)
        facts = read_model_pile(pile)
        index = SelectedModelIndex.from_snapshot(pile, facts, selector)
        cfg = Gemma4TextConfig.from_json(load_config(pile, facts, index.roots[0]))
        model = Gemma4Model(cfg, dtype=dtype, device=device)
        load_into(model, WeightLoader.from_pile(index))
        tok = None
        try:
            from ...format.tokenizer import build_tokenizer
            tok = build_tokenizer(pile, facts)
        except LookupError:
            pass
        lm = GemmaLM(model, tok, device, **kw)
        lm._pile = pile  # leaf views alias the mapping
        return lm

    from_streaming_pile = from_pile

    def complete_ids(self, ids, max_new: int, stop_on_eos: bool = False) -> list[int]:
        eos = self.engine.eos
        if not stop_on_eos:
            self.engine.eos = set()
        try:
            return self.engine.generate([list(ids)], max_new)[0]
        finally:
            self.engine.eos = eos

    def complete_multimodal(self, ids, soft_rows, soft_embeds, max_new: int, stop_on_eos: bool = True) -> list[int]:
        """Greedy continuation of a prompt whose placeholder rows ``soft_rows`` carry vision / audio soft tokens ``soft_embeds``
        (the outputs of ``Gemma4VisionTower`` / ``Gemma4AudioTower``) instead of token embeddings — the splice of
        src/models/gemma/gemma4/lm.rs:212-311 and the ``gemma_hear`` / ``gemma_listen`` loops."""
        from ...runtime.batch import BatchMeta
        seq, alloc, page = (1 << 30) - 1, self.cache.alloc, self.cache.page_size        # a sequence id the engine never hands out
        ids = [int(t) for t in ids]
        out: list[int] = []
        try:
            with torch.no_grad():
                alloc.extend(seq, len(ids))
                table, lens = alloc.page_table([seq])
                meta = BatchMeta.build([len(ids)], lens, table, page, device=self.device)
                soft = (torch.as_tensor(soft_rows, dtype=torch.long, device=self.device), soft_embeds.to(self.device))
                tok = int(self.model.greedy(torch.tensor(ids, dtype=torch.int32, device=self.device), meta, self.cache, [len(ids) - 1], soft)[0])
                while True:
                    out.append(tok)
                    if len(out) >= max_new or (stop_on_eos and tok in self.engine.eos):
                        return out
                    alloc.extend(seq, 1)
                    table, lens = alloc.page_table([seq])
                    meta = BatchMeta.build([1], lens, table, page, device=self.device)
                    tok = int(self.model.greedy(torch.tensor([tok], dtype=torch.int32, device=self.device), meta, self.cache, [0])[0])
        finally:
            alloc.release(seq)

    def complete(self, text: str, max_new: int = 128, stop: list[str] | None = None) -> str:
        if self.tokenizer is None:
            raise RuntimeError("this pile holds no tokenizer; use complete_ids")
        ids = self.tokenizer.encode(text, add_special_tokens=False).ids
        out = self.engine.generate([ids], max_new)[0]
        out = [t for t in out if t not in self.engine.eos]
        s = self.tokenizer.decode(out)
        for st in stop or []:
            if st in s:
                s = s[:s.index(st)]
        return s

    def generate(self, prompt: str, max_new: int = 128, stop: list[str] | None = None) -> str:
        return self.complete(f"<bos><|turn>user\n{prompt}<turn|>\n<|turn>model\n", max_new, stop)
