"""ctypes binding of libinquant_b200.so (declarations: include/inquant_b200.h)."""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int32, c_int64, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# INQUANT_B200_LIBRARY names a library built elsewhere (a deployment's install location)
LIBRARY_PATH = os.environ.get("INQUANT_B200_LIBRARY") or os.path.join(os.path.dirname(_HERE), "libinquant_b200.so")

F32, F16, BF16 = 0, 1, 2
DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

STATUS_NONFINITE = 1
STATUS_BAD_INDEX = 2
STATUS_WAIT_TIMEOUT = 4

OK, ERR_ARGUMENT, ERR_UNSUPPORTED, ERR_CUDA, ERR_CAPACITY = 0, -1, -2, -3, -4


class Field(ctypes.Structure):
    _fields_ = [("base", c_void_p), ("outer_stride", c_int64), ("inner_stride", c_int64)]


class Input(ctypes.Structure):
    _fields_ = [("x", c_void_p), ("dtype", c_int32), ("n_outer", c_int64), ("n_inner", c_int64),
                ("stride_outer", c_int64), ("stride_inner", c_int64), ("stride_token", c_int64),
                ("tokens", c_int32), ("channels", c_int32), ("page_ids", c_void_p), ("page_ids_i64", c_int32),
                ("num_slots", c_int64)]


class K4EncodeArgs(ctypes.Structure):
    _fields_ = [("input", Input), ("sample_stride", c_int32), ("count", c_int32), ("min_error", c_int32),
                ("payload", Field), ("scales", Field), ("salient", Field), ("donors", Field),
                ("padding", Field), ("roles", Field), ("descriptor_i32", c_int32), ("role_bytes", c_int32)]


class VEncodeArgs(ctypes.Structure):
    _fields_ = [("input", Input), ("bits", c_int32), ("group", c_int32),
                ("payload", Field), ("scales", Field), ("offsets", Field)]


class DecodeSeq(ctypes.Structure):
    _fields_ = [("query", c_void_p), ("output", c_void_p), ("query_head_stride", c_int64),
                ("table", c_void_p), ("roles", c_void_p), ("pool", c_void_p), ("page_table", c_void_p),
                ("sink_key", c_void_p), ("sink_value", c_void_p), ("tail_key", c_void_p), ("tail_value", c_void_p),
                ("sink_key_stride_h", c_int64), ("sink_key_stride_t", c_int64),
                ("sink_value_stride_h", c_int64), ("sink_value_stride_t", c_int64),
                ("tail_key_stride_h", c_int64), ("tail_key_stride_t", c_int64),
                ("tail_value_stride_h", c_int64), ("tail_value_stride_t", c_int64),
                ("n_blocks", c_int32), ("sink_tokens", c_int32), ("tail_tokens", c_int32),
                ("first_visible", c_int32), ("tail_skip", c_int32), ("pool_pages", c_int32),
                ("tail_tokens_device", c_void_p),
                ("partial_output", c_void_p), ("new_key", c_void_p), ("new_value", c_void_p),
                ("new_stride_h", c_int64), ("tail_capacity", c_int32), ("reserved", c_int32),
                ("value_roles", c_void_p)]


class DecodeArgs(ctypes.Structure):
    _fields_ = [("n_seq", c_int32), ("seqs_device", c_void_p), ("seq_host", ctypes.POINTER(DecodeSeq)),
                ("kv_heads", c_int32), ("q_per_kv", c_int32), ("block_tokens", c_int32), ("n_pad", c_int32),
                ("layout", c_int32), ("dtype", c_int32), ("scale", ctypes.c_float),
                ("page_bytes", c_int64), ("page_offsets", c_int64 * 6),
                ("pair_starts", c_void_p), ("total_units", c_int64), ("uniform_blocks", c_int32),
                ("partials", c_void_p), ("partials_floats", c_int64), ("counters", c_void_p), ("status", c_void_p),
                ("fused_append", c_int32), ("exchange_device", c_void_p), ("value_kind", c_int32), ("value_groups", c_int32)]


class DecodeExchange(ctypes.Structure):
    """``inq_decode_exchange_t``; the kernel reads it from device memory."""
    _fields_ = [("inboxes", c_void_p * 8), ("epoch", c_void_p), ("n_rows", c_int64),
                ("world", c_int32), ("rank", c_int32), ("spin_limit", c_int32), ("reserved", c_int32)]


class WritePagesArgs(ctypes.Structure):
    _fields_ = [("key_payload", c_void_p), ("key_scales", c_void_p), ("salient", c_void_p), ("donors", c_void_p),
                ("key_padding", c_void_p), ("value_payload", c_void_p), ("value_scales", c_void_p), ("value_offsets", c_void_p),
                ("pages", c_int64), ("heads", c_int32), ("block_tokens", c_int32), ("count", c_int32),
                ("pool", c_void_p), ("page_bytes", c_int64), ("page_offsets", c_int64 * 6),
                ("page_ids", c_void_p), ("page_ids_i64", c_int32), ("num_slots", c_int64), ("status", c_void_p)]


class AppendArgs(ctypes.Structure):
    _fields_ = [("key", c_void_p), ("value", c_void_p), ("src_stride_h", c_int64),
                ("tail_key", c_void_p), ("tail_value", c_void_p), ("tail_stride_h", c_int64), ("tail_stride_t", c_int64),
                ("tail_position", c_int32), ("tail_capacity", c_int32), ("tail_counter", c_void_p),
                ("sink_key", c_void_p), ("sink_value", c_void_p), ("sink_stride_h", c_int64), ("sink_stride_t", c_int64),
                ("sink_position", c_int32), ("heads", c_int32), ("row_bytes", c_int32), ("status", c_void_p)]


class RowCopy(ctypes.Structure):
    _fields_ = [("src", c_void_p), ("dst", c_void_p), ("src_stride_h", c_int64), ("src_stride_t", c_int64),
                ("dst_stride_h", c_int64), ("dst_stride_t", c_int64), ("tokens", c_int32), ("reserved", c_int32)]


class SealArgs(ctypes.Structure):
    _fields_ = [("key", ctypes.POINTER(K4EncodeArgs)), ("value_k4", ctypes.POINTER(K4EncodeArgs)),
                ("value", ctypes.POINTER(VEncodeArgs)), ("copies", RowCopy * 4),
                ("n_copies", c_int32), ("heads", c_int32), ("row_bytes", c_int32), ("reserved", c_int32)]


class GenericDecodeArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("out", c_void_p), ("q_stride_h", c_int64), ("table", c_void_p),
                ("key_roles", c_void_p), ("value_roles", c_void_p),
                ("sink_key", c_void_p), ("sink_value", c_void_p), ("tail_key", c_void_p), ("tail_value", c_void_p),
                ("sink_key_stride_h", c_int64), ("sink_key_stride_t", c_int64),
                ("sink_value_stride_h", c_int64), ("sink_value_stride_t", c_int64),
                ("tail_key_stride_h", c_int64), ("tail_key_stride_t", c_int64),
                ("tail_value_stride_h", c_int64), ("tail_value_stride_t", c_int64),
                ("n_blocks", c_int32), ("sink_tokens", c_int32), ("tail_tokens", c_int32),
                ("kv_heads", c_int32), ("q_per_kv", c_int32), ("block_tokens", c_int32), ("head_dim", c_int32),
                ("key_pad", c_int32), ("value_pad", c_int32),
                ("value_kind", c_int32), ("value_bits", c_int32), ("value_group", c_int32),
                ("dtype", c_int32), ("scale", ctypes.c_float), ("partials", c_void_p), ("partials_floats", c_int64)]


class PrefillArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("out", c_void_p),
                ("q_stride_h", c_int64), ("q_stride_t", c_int64), ("k_stride_h", c_int64), ("k_stride_t", c_int64),
                ("v_stride_h", c_int64), ("v_stride_t", c_int64), ("o_stride_h", c_int64), ("o_stride_t", c_int64),
                ("q_heads", c_int32), ("kv_heads", c_int32), ("q_tokens", c_int32), ("kv_tokens", c_int32),
                ("dtype", c_int32), ("scale", ctypes.c_float), ("status", c_void_p),
                ("workspace", c_void_p), ("workspace_bytes", c_int64)]


class ExchangeRank(ctypes.Structure):
    _fields_ = [("local", c_void_p), ("inboxes", ctypes.POINTER(c_void_p)), ("out", c_void_p),
                ("epoch", c_void_p), ("status", c_void_p), ("rank", c_int32)]


class ExchangeArgs(ctypes.Structure):
    _fields_ = [("ranks", ctypes.POINTER(ExchangeRank)), ("n_local", c_int32), ("world", c_int32),
                ("n_rows", c_int64), ("out_dtype", c_int32), ("spin_limit", c_int32)]


RECORD_FLOATS = 8 * 132  # one split-KV partial: 8 query heads x (acc[128], m, l, pad)

_lib = None


def library() -> ctypes.CDLL:
    """The shared library; raises loudly when it has not been built (there is no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIBRARY_PATH):
            raise ImportError(
                f"{LIBRARY_PATH} is missing: build it with `python inquant-open-source_b200/build.py` "
                "(nvcc, sm_100a). The packed-KV path has no Triton, PyTorch or CPU fallback.")
        lib = ctypes.CDLL(LIBRARY_PATH)
        lib.inq_last_error.restype = ctypes.c_char_p
        lib.inq_decode_workspace_floats.restype = c_int64
        lib.inq_decode_workspace_floats.argtypes = [c_int32, c_int64]
        lib.inq_decode_generic_workspace_floats.restype = c_int64
        lib.inq_decode_generic_workspace_floats.argtypes = [c_int32, c_int32, c_int32, c_int32, c_int32]
        lib.inq_prefill_workspace_bytes.restype = c_int64
        lib.inq_prefill_workspace_bytes.argtypes = [c_int32, c_int32]
        lib.inq_exchange_inbox_bytes.restype = c_int64
        lib.inq_exchange_inbox_bytes.argtypes = [c_int32, c_int64]
        lib.inq_decode_exchange_inbox_bytes.restype = c_int64
        lib.inq_decode_exchange_inbox_bytes.argtypes = [c_int32, c_int64]
        lib.inq_decode_units.restype = c_int64
        lib.inq_decode_units.argtypes = [c_int32, c_int32]
        for name in EXPORTS:
            function = getattr(lib, name)  # every declared entry point must resolve
            if name in SIGNATURES:
                function.argtypes = SIGNATURES[name]
                function.restype = c_int32
        _lib = lib
    return _lib


# Every symbol declared in include/inquant_b200.h.
EXPORTS = (
    "inq_last_error", "inq_version", "inq_k4_encode", "inq_select_donors", "inq_k4_statistics",
    "inq_k4_dequantize", "inq_k4_dequantize_strided", "inq_v_encode", "inq_v_dequantize", "inq_v_dequantize_strided",
    "inq_build_roles", "inq_write_codec_pages",
    "inq_decode_attention", "inq_decode_attention_noalloc", "inq_decode_units", "inq_merge_partials", "inq_decode_workspace_floats", "inq_append_token", "inq_append_token_batch", "inq_seal_blocks",
    "inq_prefill_attention", "inq_decode_generic", "inq_decode_generic_workspace_floats",
    "inq_prefill_workspace_bytes",
    "inq_exchange_merge", "inq_exchange_inbox_bytes", "inq_decode_exchange_inbox_bytes", "inq_restore_blocks_table", "inq_peer_buffer_create", "inq_peer_buffer_open",
    "inq_peer_buffer_close", "inq_peer_buffer_destroy",
)


_P, _I, _L = c_void_p, c_int32, c_int64
SIGNATURES = {
    "inq_k4_encode": [_P, _P, _P],
    "inq_select_donors": [_P, _P, _L, _I, _I, _P, _P, _P],
    "inq_k4_statistics": [_P, _I, _P, _P, _P, _P, _P],
    "inq_k4_dequantize": [_P, _P, _P, _P, _I, _P, _L, _I, _I, _I, _P, _I, _P],
    "inq_k4_dequantize_strided": [_P, _P, _P, _P, _I, _P, _L, _I, _I, _I, _I, _P, _L, _L, _I, _P],
    "inq_v_dequantize_strided": [_P, _P, _P, _L, _I, _I, _I, _I, _I, _P, _L, _L, _I, _P],
    "inq_v_encode": [_P, _P, _P],
    "inq_v_dequantize": [_P, _P, _P, _L, _I, _I, _I, _I, _P, _I, _P],
    "inq_build_roles": [_P, _P, _I, _L, _I, _I, _P, _I, _P],
    "inq_restore_blocks_table": [_P, _P, _I, _I, _I, _I, _P, _P, _L, _L, _I, _P],
    "inq_decode_attention": [_P, _P],
    "inq_write_codec_pages": [_P, _P],
    "inq_decode_attention_noalloc": [_P, _P],
    "inq_merge_partials": [_P, _I, _L, _P, _I, _P],
    "inq_prefill_attention": [_P, _P],
    "inq_decode_generic": [_P, _P],
    "inq_exchange_merge": [_P, _P],
    "inq_peer_buffer_create": [_L, _P, _P],
    "inq_peer_buffer_open": [_P, _P],
    "inq_peer_buffer_close": [_P],
    "inq_peer_buffer_destroy": [_P],
    "inq_append_token": [_P, _P],
    "inq_append_token_batch": [_P, _I, _P, _P],
    "inq_seal_blocks": [_P, _P, _P],
}


def check(rc: int, what: str) -> None:
    if rc == OK:
        return
    if rc == ERR_CUDA:
        raise RuntimeError(f"{what}: CUDA error: {library().inq_last_error().decode()}")
    if rc == ERR_UNSUPPORTED:
        raise NotImplementedError(f"{what}: size outside what the sm_100a kernels are built for")
    if rc == ERR_CAPACITY:
        raise ValueError(f"{what}: exceeds the fixed capacity of this entry point")
    raise ValueError(f"{what}: invalid argument")


def require_cuda(tensor: torch.Tensor, what: str) -> None:
    if tensor.device.type != "cuda":
        raise RuntimeError(f"{what} requires CUDA tensors: the B200 build has no CPU path")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_handle(device: torch.device) -> int:
    """The current CUDA stream of ``device`` as an integer handle (no stream object is built: this runs
    several times per decode call)."""
    if _raw_stream is not None:
        index = device.index
        return _raw_stream(torch.cuda.current_device() if index is None else index)
    return torch.cuda.current_stream(device).cuda_stream


def stream_identity(device: torch.device) -> tuple:
    """(device, stream handle) of the current stream, comparable across calls."""
    index = device.index
    return (torch.cuda.current_device() if index is None else index, stream_handle(device))


def stream_pointer(device: torch.device) -> c_void_p:
    return c_void_p(stream_handle(device))


_status_words: dict[torch.device, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """One zero-initialised int32 per device that kernels OR failure bits into."""
    word = _status_words.get(device)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[device] = word
    return word


def take_status(device: torch.device, mask: int = -1) -> int:
    """Read the status word and clear the bits of ``mask`` that were set (synchronises the current
    stream).  Bits outside ``mask`` stay in the word for whoever asks for them: a wait that timed
    out or a skipped index is not lost because an encoder checked its finite bit in between.
    Returns the bits of ``mask`` that were set."""
    word = status_word(device)
    value = int(word.item()) & mask
    if value:
        word.bitwise_and_(~value)
    return value


_deferred_depth = 0


class deferred_status:
    """Inside this context the encoders do not read the status word after a launch (no stream
    synchronisation); failure bits stay in the word until ``take_status`` is called."""

    def __enter__(self):
        global _deferred_depth
        _deferred_depth += 1
        return self

    def __exit__(self, *_exc):
        global _deferred_depth
        _deferred_depth -= 1


def nonfinite_reported(device: torch.device) -> bool:
    """The encoders' finite check: reads and clears the status word (a synchronisation) unless
    status reads are deferred."""
    if _deferred_depth:
        return False
    return bool(take_status(device, STATUS_NONFINITE))


def pointer(tensor: torch.Tensor | None) -> c_void_p:
    return c_void_p(None if tensor is None or tensor.numel() == 0 else tensor.data_ptr())


def compact_field(tensor: torch.Tensor | None, n_inner: int) -> Field:
    """Field descriptor of a contiguous tensor whose two leading axes are (outer, inner)."""
    if tensor is None or tensor.numel() == 0:
        return Field(None, 0, 0)
    row = tensor.element_size()
    for size in tensor.shape[2:]:   # plain integers: indexing the tensor costs four times as much
        row *= size
    return Field(tensor.data_ptr(), row * n_inner, row)


def make_input(x: torch.Tensor, page_ids: torch.Tensor | None = None, num_slots: int = 0) -> Input:
    """``x`` is [outer, inner, tokens, channels] with unit channel stride (any other strides).
    ``num_slots`` is the number of rows of the destination that ``page_ids`` index (ids outside it
    are skipped on the device and reported through the status word)."""
    assert x.ndim == 4 and x.stride(3) == 1
    return Input(x.data_ptr(), DTYPE_CODE[x.dtype], x.shape[0], x.shape[1], x.stride(0), x.stride(1), x.stride(2),
                 x.shape[2], x.shape[3], None if page_ids is None else page_ids.data_ptr(),
                 0 if page_ids is None else int(page_ids.dtype == torch.int64), int(num_slots))


_counters: dict[tuple, torch.Tensor] = {}


def decode_counters(device: torch.device, count: int) -> torch.Tensor:
    """Zero-initialised arrival counters of the fused split-KV merge, one array per
    (device, stream); the kernel leaves them zero, so they are reused launch after launch."""
    key = (device, stream_handle(device))
    tensor = _counters.get(key)
    if tensor is None or tensor.numel() < count + 1:   # one more: the launch-wide arrival counter of a fused append
        tensor = torch.zeros(max(count + 1, 1024), dtype=torch.int32, device=device)
        _counters[key] = tensor
    return tensor


def dense_rows_aligned(tensor: torch.Tensor) -> bool:
    """16-byte aligned rows of a [1, heads, tokens, 128] 16-bit tensor."""
    return (tensor.data_ptr() % 16 == 0 and tensor.stride(-1) == 1 and tensor.stride(1) % 8 == 0
            and tensor.stride(2) % 8 == 0)
