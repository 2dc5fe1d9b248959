"""Attribute ids of the model-graph format.

The ids are the reference's, so that facts written by either side name the same attributes
(src/format.rs:52-127, src/leaf.rs:51-61, src/models/inkling/pile.rs:416-464,
src/jsonfacts.rs:55-102, src/models/gemma/lora.rs:43-53).
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


# The storage crate's own metadata namespace (`metadata::tag`, `metadata::name`) is not part of the reference tree, so its two
# attribute ids cannot be read there; these stand-ins are derived from the names.
META_TAG = derived_id(b"triblespace.metadata", b"tag")
META_NAME = derived_id(b"triblespace.metadata", b"name")
# JSON documents as facts (src/jsonfacts.rs:55-102): nine attributes — member and index are the format's own (reused, same
# encodings), six are minted there, and node types are `metadata::tag` discriminants
JSON_KEY = id_hex("051B238236962081B98F5D44BD9FA999")        # Handle<UTF8>: an object member's key
JSON_STRING = id_hex("65D08DFB670E7E3729BE6BC2C0073CAD")     # Handle<UTF8>
JSON_INT = id_hex("8657CA9A8F2864E21FA1793AF47AACA2")        # I256BE
JSON_FLOAT = id_hex("3B3EC066DE93041ACB2A26709CD11017")      # F64
JSON_BOOL = id_hex("AB52DBDC419DE0ECC7D56632D7B29B61")       # Boolean
DOCUMENT_ROOT = id_hex("C3BE4C8C259D1A1C1BB2BF8C19DF41F3")   # GenId: document node -> JSON root
JSON_OBJECT = id_hex("0956A91F3198144BC1E1920467F9CE1A")     # type tags (src/jsonfacts.rs:55-70)
JSON_ARRAY = id_hex("3DDDE71CF6B902D3CE15ABF3B3FE9A06")
JSON_NULL = id_hex("CBD6C0C8FD1DA5A4851429ABAE3CFA9F")
JSON_DOCUMENT = id_hex("686F919B71279386F31EB34A389E3241")
# LoRA adapters (src/models/gemma/lora.rs:43-53)
LORA_RANK = id_hex("1A682F45CE40171DD5C6FDB4F086AD69")       # U256BE
LORA_ALPHA = id_hex("198B03AF556B7505CCC9ABD4A1D6E724")      # F64
LORA_ADAPTER = id_hex("B93C4E66F4B9553BF0E8B5DBAD116ECF")    # GenId, repeated on the LoRA set entity
LORA_PROJECTION = id_hex("FF8335C187823A267E26B4E33EF157E9") # ShortString
LORA_A = id_hex("7CD7F0DC8BDA328735A22DF02B4B8828")          # Handle<F32Array> [rank, in]
LORA_B = id_hex("1F21DAE68652A4D8CAD973400F04124D")          # Handle<F32Array> [out, rank]
# training-state checkpoint (this build: optimizer moments, step, RNG)
TRAIN_STEP = derived_id(b"mary_b200.train", b"step")
TRAIN_STATE = derived_id(b"mary_b200.train", b"state_blob")
TRAIN_RUN = derived_id(b"mary_b200.train", b"run")
TRAIN_ADAPTER = derived_id(b"mary_b200.train", b"adapter")

KINDS = ("vector", "matrix", "conv", "tensor")
# ownership label that ties a document or tokenizer to a model root (MODEL_ROOT marks roots only)
OWNER = derived_id(b"mary_b200.schema", b"owner")
