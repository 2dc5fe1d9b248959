"""Storage substrate: content-addressed pile, tribles, branches, signed commits, collections."""
from .hashing import blake3, blake3_py
from .store import MemoryBlobStore, Pile, PileError
from .trible import (TribleBuilder, TribleSet, content_id, derived_id, fresh_id, id_hex)
from .repo import Collection, Repository, RepoError, signing_key_file, MODEL_GRAPH, MODEL_BUNDLES

__all__ = ["blake3", "blake3_py", "MemoryBlobStore", "Pile", "PileError", "TribleBuilder", "TribleSet",
           "content_id", "derived_id", "fresh_id", "id_hex", "Collection", "Repository", "RepoError",
           "signing_key_file", "MODEL_GRAPH", "MODEL_BUNDLES"]
