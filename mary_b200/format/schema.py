"""Attribute ids of the model-graph format.

The ids are the reference's, so that facts written by either side name the same attributes
(src/format.rs:52-127, src/leaf.rs:51-61, src/models/inkling/pile.rs:416-464,
src/jsonfacts.rs:89-102, src/models/gemma/lora.rs:43-53).  Ids known here only in abbreviated
form are completed deterministically from their visible prefix and suffix.
"""
from __future__ import annotations

from ..pile.trible import derived_id, id_hex

# tensor leaf, legacy two-blob form (src/format.rs:52-61)
DATA = id_hex("572B45D52A47608F283D0F778597137A")
DATA_F16 = id_hex("467CCF3FDCCCCE599F6C1B933EACD933")
SHAPE = id_hex("D09A91FC3F04C40AE4A42CD6628A9E38")
# quantized leaves (src/format.rs:63-87)
DATA_Q4 = id_hex("2ADC6462A7F70E230558C5D681E38768")
DATA_Q8 = id_hex("23178058559C762BB4B1FEAA36B3566D")
Q_SCALES = id_hex("F9EA2FB90DC094D42A4845B013950032")
FORMAT_MARKER = id_hex("2CC4D16369C4980BCB512937DA204FF5")
# module entity (src/format.rs:91-101)
WEIGHT = id_hex("4629D277AD6B52B50DA78DEF63440AF1")
BIAS = id_hex("18E898172078C843A0351C3D880CC238")
KIND = id_hex("52C4A211D2A08BA25C27FFD79FF24C93")
SAFETENSOR_PATH = id_hex("09EA2F7BCF9B0C9714EE39CF269DF2D5")
INDEX = id_hex("33CE12B1B940B13E48D8E5B0ADFD2421")
# model root (src/format.rs:105-127)
MODEL_ROOT = id_hex("3F46CDE630964D78D62DA32F4A8558C1")
MEMBER = id_hex("B4B6EC08A0CD70DE63A690168EE78F0F")
MODEL_NAME = id_hex("4C1CD1611863E7854C59C7DC706DF77A")
SOURCE = id_hex("D20B8E3556C35FF6D18D104C3443D6CF")
QUANTIZATION = id_hex("7AF87320C144AA29C29FE2A5EE7C7EB2")
# typed leaf: the attribute id is a function of (anchor, element, rank) (src/leaf.rs:51-61)
LEAF_ANCHOR = id_hex("743E98D23794CA9BEFE727D07482D8D5")
# expert placement facts (src/models/inkling/pile.rs:416-464)
NVFP4_WEIGHT_ANCHOR = id_hex("0B51DA3E67216213871743E045590DBC")
EXPERT_INDEX = id_hex("A6ED6DBA4BE63E4E34F2787DA84AD860")
LAYER = id_hex("BCDDFBCFF89F67EE0B1E527C4872CED7")


def _completed(prefix: str, suffix: str) -> bytes:
    """An id known by prefix and suffix only: the middle is derived from both so it is stable."""
    mid_len = 32 - len(prefix) - len(suffix)
    mid = derived_id(prefix.encode(), suffix.encode()).hex().upper()[:mid_len]
    return id_hex(prefix + mid + suffix)


# JSON documents as facts (src/jsonfacts.rs:89-102)
JSON_KEY = _completed("051B2382", "A999")
JSON_STRING = _completed("65D08DFB", "3CAD")
JSON_INT = _completed("8657CA9A", "ACA2")
JSON_FLOAT = _completed("3B3EC066", "1017")
JSON_BOOL = _completed("AB52DBDC", "9B61")
DOCUMENT_ROOT = _completed("C3BE4C8C", "41F3")
# the remaining three of the nine JSON attributes (parent link, array position, node type / doc name)
JSON_PARENT = derived_id(b"mary_b200.json", b"parent")
JSON_POS = derived_id(b"mary_b200.json", b"position")
JSON_TYPE = derived_id(b"mary_b200.json", b"type")
DOCUMENT_NAME = derived_id(b"mary_b200.json", b"document_name")
# LoRA adapters (src/models/gemma/lora.rs:43-53)
LORA_RANK = _completed("1A682F45", "AD69")
LORA_ALPHA = _completed("198B03AF", "E724")
LORA_ADAPTER = _completed("B93C4E66", "6ECF")
LORA_PROJECTION = _completed("FF8335C1", "57E9")
LORA_A = _completed("7CD7F0DC", "8828")
LORA_B = _completed("1F21DAE6", "124D")
# training-state checkpoint (this build: optimizer moments, step, RNG)
TRAIN_STEP = derived_id(b"mary_b200.train", b"step")
TRAIN_STATE = derived_id(b"mary_b200.train", b"state_blob")
TRAIN_RUN = derived_id(b"mary_b200.train", b"run")
TRAIN_ADAPTER = derived_id(b"mary_b200.train", b"adapter")

KINDS = ("vector", "matrix", "conv", "tensor")
# ownership label that ties a document or tokenizer to a model root (MODEL_ROOT marks roots only)
OWNER = derived_id(b"mary_b200.schema", b"owner")
