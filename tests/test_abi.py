"""The C-ABI library loads and exports every symbol the header declares (no GPU needed)."""
import ctypes
import os
import re

from unified_cache_management_b200 import build as ucm_build
from unified_cache_management_b200 import lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "ucmr.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ucmr_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    path = ucm_build.build_library()
    names = _declared()
    assert len(names) >= 14
    lib = ctypes.CDLL(path)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in ucmr.h but not exported"
        assert n in L.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(L.SIGNATURES) == names


def test_version_and_status_strings():
    lib = L.load_library()
    assert lib.ucmr_version() == 100
    assert lib.ucmr_status_string(0) == b"ok"
    assert b"workspace" in lib.ucmr_status_string(L.UCMR_ERR_WORKSPACE)
    assert lib.ucmr_hamming_topk_workspace_bytes(16, 8, 1024, 0) == L.WORKSPACE_HEADER_BYTES + 16 * 8 * 1024 * 4
    assert lib.ucmr_hamming_topk_workspace_bytes(16, 8, 1024, 1) == L.WORKSPACE_HEADER_BYTES + 16 * 1024 * 4
    # one kv head: room for the query planes of the token-row scan on top
    assert lib.ucmr_hamming_topk_workspace_bytes(16, 1, 1024, 0) > L.WORKSPACE_HEADER_BYTES + 16 * 1024 * 4


def test_host_argument_validation_needs_no_gpu():
    """Entry points reject bad arguments before touching the device."""
    lib = L.load_library()
    null = ctypes.c_void_p(0)
    assert lib.ucmr_update_seq_lens(null, 4, 128, 128, null, null) == L.UCMR_ERR_BAD_ARG
    assert lib.ucmr_merge_topk(null, null, 0, 1, 1, 1, 1, 1, null, null, null) == L.UCMR_ERR_BAD_ARG
    assert lib.ucmr_gather_kv(null, null, 1, 16, null, 1, 1, 0, 1, 1, 16, null, null, null, null) == L.UCMR_ERR_BAD_ARG
    assert lib.ucmr_hash_encode(null, 1, 128, null, 128, 128, null, null, null) == L.UCMR_ERR_BAD_ARG
    assert lib.ucmr_workspace_init(null, 0, null) == L.UCMR_ERR_WORKSPACE
    # the step timeline only exists in the trace build
    stamps = (ctypes.c_ulonglong * 32)()
    assert lib.ucmr_trace_read(0, null) == L.UCMR_ERR_BAD_ARG
    assert lib.ucmr_trace_read(0, ctypes.cast(stamps, ctypes.c_void_p)) == L.UCMR_ERR_UNSUPPORTED
