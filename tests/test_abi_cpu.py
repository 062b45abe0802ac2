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
    assert ctypes.sizeof(N.DecodeSeq) == 232
    assert ctypes.sizeof(N.PrefillArgs) == 4 * 8 + 8 * 8 + 4 * 4 + 4 + 4 + 8 + 8 + 8
    assert ctypes.sizeof(N.GenericDecodeArgs) % 8 == 0
    assert ctypes.sizeof(N.ExchangeRank) == 48 and ctypes.sizeof(N.ExchangeArgs) == 32


def test_struct_mirrors_match_the_header_as_a_c_compiler_lays_it_out(tmp_path):
    """sizeof and the offsets of the bounds fields (pool_pages, num_slots), taken from the header
    by gcc, equal those of the ctypes mirrors."""
    import subprocess
    from inquant import _native as N
    structs = [("inq_field_t", N.Field), ("inq_input_t", N.Input), ("inq_k4_encode_args_t", N.K4EncodeArgs),
               ("inq_v_encode_args_t", N.VEncodeArgs), ("inq_decode_seq_t", N.DecodeSeq),
               ("inq_decode_args_t", N.DecodeArgs), ("inq_append_args_t", N.AppendArgs),
               ("inq_decode_generic_args_t", N.GenericDecodeArgs), ("inq_prefill_args_t", N.PrefillArgs),
               ("inq_exchange_rank_t", N.ExchangeRank), ("inq_exchange_args_t", N.ExchangeArgs),
               ("inq_decode_exchange_t", N.DecodeExchange), ("inq_row_copy_t", N.RowCopy),
               ("inq_seal_args_t", N.SealArgs)]
    offsets = [("inq_input_t", "num_slots", N.Input.num_slots.offset),
               ("inq_decode_seq_t", "pool_pages", N.DecodeSeq.pool_pages.offset),
               ("inq_decode_seq_t", "tail_tokens_device", N.DecodeSeq.tail_tokens_device.offset),
               ("inq_decode_seq_t", "partial_output", N.DecodeSeq.partial_output.offset),
               ("inq_decode_args_t", "exchange_device", N.DecodeArgs.exchange_device.offset),
               ("inq_decode_exchange_t", "n_rows", N.DecodeExchange.n_rows.offset),
               ("inq_seal_args_t", "n_copies", N.SealArgs.n_copies.offset)]
    lines = ["#include <stdio.h>", "#include <stddef.h>", f'#include "{HEADER}"', "int main(void) {"]
    lines += [f'  printf("%zu\\n", sizeof({name}));' for name, _ in structs]
    lines += [f'  printf("%zu\\n", offsetof({name}, {field}));' for name, field, _ in offsets]
    lines += ["  return 0;", "}"]
    source = tmp_path / "sizes.c"
    source.write_text("\n".join(lines))
    binary = tmp_path / "sizes"
    subprocess.run(["gcc", "-std=c11", str(source), "-o", str(binary)], check=True)
    got = [int(x) for x in subprocess.run([str(binary)], check=True, capture_output=True, text=True).stdout.split()]
    want = [ctypes.sizeof(mirror) for _, mirror in structs] + [offset for _, _, offset in offsets]
    assert got == want


def test_exchange_entry_points_check_their_arguments_without_a_gpu():
    from inquant import _native as N
    lib = N.library()
    assert lib.inq_exchange_inbox_bytes(9, 10) == 0 and lib.inq_exchange_inbox_bytes(2, 0) == 0
    assert lib.inq_exchange_inbox_bytes(2, 10) == 2 * 8 * 512 * 4 + 2 * 2 * 10 * 520
    assert lib.inq_decode_exchange_inbox_bytes(2, 10) == 2 * 8 * 512 * 4 + 2 * 2 * 10 * 1040
    assert lib.inq_decode_exchange_inbox_bytes(0, 10) == 0
    args = N.ExchangeArgs(None, 1, 2, 10, 2, 0)
    assert lib.inq_exchange_merge(ctypes.byref(args), None) == N.ERR_ARGUMENT
    assert lib.inq_peer_buffer_create(0, None, None) == N.ERR_ARGUMENT
    assert lib.inq_peer_buffer_open(None, None) == N.ERR_ARGUMENT
    assert lib.inq_peer_buffer_close(None) == N.ERR_ARGUMENT and lib.inq_peer_buffer_destroy(None) == N.ERR_ARGUMENT


def test_seal_entry_point_refuses_bad_row_copies_before_any_launch():
    """`inq_seal_blocks` checks every argument before its first launch, so a refused call needs no GPU."""
    from inquant import _native as N
    lib = N.library()
    word = ctypes.c_int32(0)
    status = ctypes.cast(ctypes.pointer(word), ctypes.c_void_p)
    assert lib.inq_seal_blocks(None, status, None) == N.ERR_ARGUMENT
    args = N.SealArgs()
    assert lib.inq_seal_blocks(ctypes.byref(args), None, None) == N.ERR_ARGUMENT
    args.n_copies = 5
    assert lib.inq_seal_blocks(ctypes.byref(args), status, None) == N.ERR_ARGUMENT
    args.n_copies, args.heads, args.row_bytes = 1, 4, 250          # rows are not whole 16-byte vectors
    assert lib.inq_seal_blocks(ctypes.byref(args), status, None) == N.ERR_ARGUMENT
    args.row_bytes = 256
    args.copies[0].src, args.copies[0].dst, args.copies[0].tokens = 4096, 8200, 3   # destination not 16-byte aligned
    assert lib.inq_seal_blocks(ctypes.byref(args), status, None) == N.ERR_ARGUMENT
    args.copies[0].dst, args.copies[0].src_stride_t = 8192, 250
    assert lib.inq_seal_blocks(ctypes.byref(args), status, None) == N.ERR_ARGUMENT
    # nothing to encode and nothing to copy is a valid call that launches nothing
    assert lib.inq_seal_blocks(ctypes.byref(N.SealArgs()), status, None) == N.OK
