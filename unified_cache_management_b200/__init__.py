"""B200-native hash-code top-k block retrieval (the sparse-attention retrieval path of UCM).

The compute lives in ``libucmr_b200.so`` (hand-written sm_100a CUDA behind the C ABI declared in
``include/ucmr.h``); this package is the thin Python host side that mirrors the reference
project's operator and plugin interfaces for that path.  There is no CPU fallback: importing the
ops without the built library raises.
"""
from .lib import UcmrError, library_path, load_library  # noqa: F401

__all__ = ["UcmrError", "library_path", "load_library"]
