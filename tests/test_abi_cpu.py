"""The C-ABI library builds, loads without a GPU and exports every entry point that
include/inquant_b200.h declares (no compute calls here)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "inquant_b200.h")


def _declared_functions():
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    text = re.sub(r"typedef\s+struct\s*\{.*?\}\s*\w+\s*;", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(inq_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = _declared_functions()
    for required in ("inq_k4_encode", "inq_v_encode", "inq_select_donors", "inq_append_token",
                     "inq_decode_attention", "inq_merge_partials", "inq_prefill_attention", "inq_decode_generic"):
        assert required in names


def test_library_loads_and_exports_every_declared_symbol():
    import sys
    sys.path.insert(0, os.path.join(ROOT, "inquant-open-source_b200"))
    import build
    path = build.build_library()
    lib = ctypes.CDLL(path)
    for name in _declared_functions():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    lib.inq_version.restype = ctypes.c_int
    assert lib.inq_version() > 0


def test_python_binding_lists_the_same_symbols():
    from inquant import _native
    assert sorted(_native.EXPORTS) == _declared_functions()


def test_struct_mirrors_have_the_sizes_the_header_implies():
    from inquant import _native as N
    assert ctypes.sizeof(N.DecodeSeq) == 192
    assert ctypes.sizeof(N.PrefillArgs) == 4 * 8 + 8 * 8 + 4 * 4 + 4 + 4 + 8 + 8 + 8
    assert ctypes.sizeof(N.GenericDecodeArgs) % 8 == 0
    assert ctypes.sizeof(N.ExchangeRank) == 48 and ctypes.sizeof(N.ExchangeArgs) == 32


def test_exchange_entry_points_check_their_arguments_without_a_gpu():
    from inquant import _native as N
    lib = N.library()
    assert lib.inq_exchange_inbox_bytes(9, 10) == 0 and lib.inq_exchange_inbox_bytes(2, 0) == 0
    assert lib.inq_exchange_inbox_bytes(2, 10) == 2 * 8 * 512 * 4 + 2 * 2 * 10 * 520
    args = N.ExchangeArgs(None, 1, 2, 10, 2, 0)
    assert lib.inq_exchange_merge(ctypes.byref(args), None) == N.ERR_ARGUMENT
    assert lib.inq_peer_buffer_create(0, None, None) == N.ERR_ARGUMENT
    assert lib.inq_peer_buffer_open(None, None) == N.ERR_ARGUMENT
    assert lib.inq_peer_buffer_close(None) == N.ERR_ARGUMENT and lib.inq_peer_buffer_destroy(None) == N.ERR_ARGUMENT
