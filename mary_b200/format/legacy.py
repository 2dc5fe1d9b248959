"""Projection between the two generations of model-graph attribute ids.

Reference: src/model_collection.rs:897-1322.  Model piles written before the reference's "attribute epoch" name their attributes by
LITERAL 16-byte ids (the 45 below: tensor format, model graph, Gemma LoRA, tokenizer graph).  Later runtime declarations derive the
id from the same hex string used as an ANCHOR together with the attribute's value encoding, so one fact can be stored under either
id.  ``project_legacy_model_attributes`` makes a fact set readable by both generations: it is strictly additive (every input
trible is kept, unknown attributes are untouched, the alias ``(entity, canonical attribute, value)`` is inserted only when
missing), so running it over its own result adds nothing, and it reports per-attribute counts.

This package writes and reads the LITERAL ids (``format.schema``, ``format.tokenizer``), i.e. the historical side of the table, so
its piles are what the reference's own projection upgrades.  ``project_to_literal`` is the opposite direction: it lets the loaders
here read a fact set that carries only derived ids.  The derivation itself lives in the reference's triple-store crate, whose
source is not part of the reference tree; ``anchored_id`` below is a stand-in with the two properties the projection relies on
(a pure function of anchor and value encoding; disjoint from every literal id, so no ``A -> B -> C`` chain can arise) and is the
one place to change once the real derivation is known."""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from ..pile.trible import TribleSet, derived_id, id_hex

# (label, literal id, value encoding) — src/model_collection.rs:946-1008
_TABLE = (
    ("format.data", "572B45D52A47608F283D0F778597137A", "Handle<F32Array>"),
    ("format.data_f16", "467CCF3FDCCCCE599F6C1B933EACD933", "Handle<F16Array>"),
    ("format.shape", "D09A91FC3F04C40AE4A42CD6628A9E38", "Handle<U64Array>"),
    ("format.data_q4", "2ADC6462A7F70E230558C5D681E38768", "Handle<U32Array>"),
    ("format.data_q8", "23178058559C762BB4B1FEAA36B3566D", "Handle<U32Array>"),
    ("format.q_scales", "F9EA2FB90DC094D42A4845B013950032", "Handle<F16Array>"),
    ("format.format_marker", "2CC4D16369C4980BCB512937DA204FF5", "GenId"),
    ("format.weight", "4629D277AD6B52B50DA78DEF63440AF1", "GenId"),
    ("format.bias", "18E898172078C843A0351C3D880CC238", "GenId"),
    ("format.kind", "52C4A211D2A08BA25C27FFD79FF24C93", "ShortString"),
    ("format.safetensor_path", "09EA2F7BCF9B0C9714EE39CF269DF2D5", "Handle<UTF8String>"),
    ("format.index", "33CE12B1B940B13E48D8E5B0ADFD2421", "U256BE"),
    ("format.model_root", "3F46CDE630964D78D62DA32F4A8558C1", "GenId"),
    ("format.member", "B4B6EC08A0CD70DE63A690168EE78F0F", "GenId"),
    ("format.model_name", "4C1CD1611863E7854C59C7DC706DF77A", "Handle<UTF8String>"),
    ("format.source", "D20B8E3556C35FF6D18D104C3443D6CF", "Handle<UTF8String>"),
    ("format.quantization", "7AF87320C144AA29C29FE2A5EE7C7EB2", "ShortString"),
    ("gemma_lora.lora_rank", "1A682F45CE40171DD5C6FDB4F086AD69", "U256BE"),
    ("gemma_lora.lora_alpha", "198B03AF556B7505CCC9ABD4A1D6E724", "F64"),
    ("gemma_lora.lora_adapter", "B93C4E66F4B9553BF0E8B5DBAD116ECF", "GenId"),
    ("gemma_lora.lora_projection", "FF8335C187823A267E26B4E33EF157E9", "ShortString"),
    ("gemma_lora.lora_a", "7CD7F0DC8BDA328735A22DF02B4B8828", "Handle<F32Array>"),
    ("gemma_lora.lora_b", "1F21DAE68652A4D8CAD973400F04124D", "Handle<F32Array>"),
    ("tokenizer.tokenizer", "E7014108A8F9512B19E3E8272E8A71F9", "GenId"),
    ("tokenizer.vocab", "E839AA8F549C0D608FB86476A1EF3416", "GenId"),
    ("tokenizer.merge", "E229769197BB035A2D6F61BC6A7D44BC", "GenId"),
    ("tokenizer.added", "B2553118F4CAAF1D028619956DE7F145", "GenId"),
    ("tokenizer.normalizer", "53BAF87A0E7F1410F8212B3EDF2A498C", "GenId"),
    ("tokenizer.pre_tokenizer", "6EEBF39CADD11B7CFBB624019AE21585", "GenId"),
    ("tokenizer.post_processor", "98EC58B28F4D0BB43965DF7C5FF22713", "GenId"),
    ("tokenizer.decoder", "F3AAA4CD8EE04E5592059564A21FE953", "GenId"),
    ("tokenizer.piece", "AE7FE29F2F38153F58C542D5CA4A9356", "Handle<UTF8String>"),
    ("tokenizer.token_id", "F0E2E782F7BB62F52B1186DDE0EB5388", "U256BE"),
    ("tokenizer.piece_bytes", "714AE13F801202EB27C83E3AB2290669", "Handle<RawBytes>"),
    ("tokenizer.merge_left", "5723ECE1FF426C58879B79D5669A7CF1", "Handle<UTF8String>"),
    ("tokenizer.merge_right", "5C78FEB151F35A2C5D07BEC92E860752", "Handle<UTF8String>"),
    ("tokenizer.unk_token", "68F1A9E6ED735E7C3ADCCA076AFF1742", "ShortString"),
    ("tokenizer.continuing_subword_prefix", "11F76A2C0856C16CB030C4327D5A3B93", "ShortString"),
    ("tokenizer.end_of_word_suffix", "6FB969E8A3EDD1A657C721DD5A7D42EA", "ShortString"),
    ("tokenizer.max_input_chars", "DF3F88DBFA2B44A7783169C9640014AF", "U256BE"),
    ("tokenizer.piece_score", "3BCB70478942DB710ED2A4FB023F3457", "F64"),
    ("tokenizer.byte_fallback", "EE4C6647619A836326196F0DBF84FA98", "Boolean"),
    ("tokenizer.pattern", "C8262D5668B8A1F541B3C35D54201BEC", "Handle<UTF8String>"),
    ("tokenizer.replace_content", "3AC7574C07D02D389B4E7AD3B3B084D9", "ShortString"),
    ("tokenizer.behavior", "964B4FCF7477E7E4436F0325F89B7CB5", "ShortString"),
)
LEGACY_MODEL_ATTRIBUTE_ALIAS_COUNT = 45


def anchored_id(anchor_hex: str, encoding: str) -> bytes:
    """Stand-in for the derived (anchor + value encoding) attribute id; see the module text."""
    return derived_id(b"anchored-attribute", id_hex(anchor_hex), encoding.encode())


@dataclass(frozen=True)
class ModelAttributeAlias:
    label: str
    historical: bytes
    canonical: bytes


@dataclass
class AliasCounts:
    alias: ModelAttributeAlias
    source_facts: int = 0
    aliases_added: int = 0
    aliases_already_present: int = 0


@dataclass
class Projection:
    facts: TribleSet
    input_facts: int
    source_facts: int = 0
    aliases_added: int = 0
    mappings: list = field(default_factory=list)


def legacy_model_attribute_aliases() -> list[ModelAttributeAlias]:
    out = [ModelAttributeAlias(label, id_hex(h), anchored_id(h, enc)) for label, h, enc in _TABLE]
    hist, canon = {a.historical for a in out}, {a.canonical for a in out}
    if len(out) != LEGACY_MODEL_ATTRIBUTE_ALIAS_COUNT or len(hist) != len(out) or len(canon) != len(out) or hist & canon:
        raise AssertionError("alias table must hold 45 distinct literal ids and 45 distinct derived ids, disjoint from one another")
    return out


def _project(facts: TribleSet, forward: bool) -> Projection:
    aliases = legacy_model_attribute_aliases()
    counts = [AliasCounts(a) for a in aliases]
    by_src = {(a.historical if forward else a.canonical): i for i, a in enumerate(aliases)}
    have = {bytes(r) for r in facts.data} if len(facts) else set()
    new_rows = []
    proj = Projection(facts, len(facts), mappings=counts)
    for row in (facts.data if len(facts) else ()):
        b = bytes(row)
        i = by_src.get(b[16:32])
        if i is None:
            continue
        c = counts[i]
        c.source_facts += 1
        proj.source_facts += 1
        alias = b[:16] + (c.alias.canonical if forward else c.alias.historical) + b[32:]
        if alias in have:
            c.aliases_already_present += 1
        else:
            have.add(alias)
            new_rows.append(alias)
            c.aliases_added += 1
            proj.aliases_added += 1
    if new_rows:
        extra = TribleSet(np.frombuffer(b"".join(new_rows), dtype=np.uint8).reshape(-1, 64).copy())
        proj.facts = facts | extra
    return proj


def project_legacy_model_attributes(facts: TribleSet) -> Projection:
    """Add the derived-id alias of every literal-id fact (src/model_collection.rs:1258-1313)."""
    return _project(facts, True)


def project_to_literal(facts: TribleSet) -> Projection:
    """The opposite direction: add the literal-id alias of every derived-id fact, so that this package's loaders can read it."""
    return _project(facts, False)
