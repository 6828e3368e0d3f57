"""ctypes binding of ``libitak_cuda_compute.so`` (the C ABI of include/itak_cuda_compute.h)."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(HERE, "lib", "libitak_cuda_compute.so")

# itk_status
OK = 0
ERR_ZERO_DIMENSION = 1
ERR_INVALID_WINDOW = 2
ERR_SIZE_OVERFLOW = 3
ERR_SHAPE_MISMATCH = 4
ERR_INVALID_LAYER = 5
ERR_OUT_OF_ORDER_POSITION = 6
ERR_NON_DIVISIBLE_HEADS = 7
ERR_NO_VISIBLE_KEYS = 8
ERR_CHECKPOINT_BUSY = 9
ERR_STALE_CHECKPOINT = 10
ERR_CHECKPOINT_TOO_DEEP = 11
ERR_CHECKPOINT_RANGE_EXCEEDED = 12
ERR_BULK_RESTORE_NOT_FRESH = 13
ERR_REWIND_OUT_OF_RANGE = 14
ERR_INCOHERENT_CACHE = 32
ERR_INCONSISTENT_SNAPSHOT = 33
ERR_BAD_MAGIC = 34
ERR_UNSUPPORTED_VERSION = 35
ERR_TRUNCATED = 36
ERR_CHECKSUM_MISMATCH = 37
ERR_GEOMETRY_MISMATCH = 38
ERR_FINGERPRINT_MISMATCH = 39
ERR_EMPTY_PREFIX = 40
ERR_TOKEN_COUNT_MISMATCH = 41
ERR_PREFIX_HASH_MISMATCH = 42
ERR_SNAPSHOT_TOKEN_MISMATCH = 43
ERR_ENTRY_TOO_LARGE = 44
ERR_INVALID_CONFIG = 45
ERR_IO = 46
ERR_STEP_FAILED = 64
ERR_CUDA = 100
ERR_INVALID_ARGUMENT = 101
ERR_CAPACITY = 102
ERR_INVALID_SLOT = 103

KV_F32 = 0
KV_F16 = 1


class Config(C.Structure):
    _fields_ = [
        ("n_layers", C.c_uint32),
        ("layer_window", C.POINTER(C.c_uint32)),
        ("q_heads", C.c_uint32),
        ("kv_heads", C.c_uint32),
        ("head_dim", C.c_uint32),
        ("n_slots", C.c_uint32),
        ("max_context", C.c_uint32),
        ("chunk_cap", C.c_uint32),
        ("kv_dtype", C.c_int32),
        ("device", C.c_int32),
    ]


class Checkpoint(C.Structure):
    _fields_ = [
        ("id", C.c_uint64),
        ("serial", C.c_uint64),
        ("base", C.c_uint64),
        ("max_round_tokens", C.c_uint64),
    ]


class PrepConfig(C.Structure):
    _fields_ = [
        ("q_norm_weight", C.POINTER(C.c_float)),
        ("k_norm_weight", C.POINTER(C.c_float)),
        ("norm_eps", C.c_float),
        ("rope_base", C.c_float),
        ("rotary_dim", C.c_uint32),
        ("pairing", C.c_uint32),
    ]


class Stats(C.Structure):
    _fields_ = [
        ("attention_calls", C.c_uint64),
        ("kernel_launches", C.c_uint64),
        ("rows_appended", C.c_uint64),
        ("kv_bytes_read", C.c_uint64),
        ("prefix_captures", C.c_uint64),
        ("prefix_restores", C.c_uint64),
        ("last_splits", C.c_uint64),
    ]


_u32, _u64, _sz, _vp = C.c_uint32, C.c_uint64, C.c_size_t, C.c_void_p
_fp = C.POINTER(C.c_float)
_u32p, _u64p = C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)

# name -> (restype, argtypes): every entry point include/itak_cuda_compute.h declares.
SIGNATURES = {
    "itk_backend_create": (C.c_int, [C.POINTER(Config), C.POINTER(_vp)]),
    "itk_backend_destroy": (None, [_vp]),
    "itk_last_error": (C.c_char_p, [_vp]),
    "itk_set_stream": (C.c_int, [_vp, _vp]),
    "itk_set_option": (C.c_int, [_vp, C.c_char_p, C.c_int64]),
    "itk_synchronize": (C.c_int, [_vp]),
    "itk_get_stats": (C.c_int, [_vp, C.POINTER(Stats)]),
    "itk_attention": (C.c_int, [_vp, _u32, _u32, _vp, _sz, _vp, _sz, _vp, _sz, _u64, _vp]),
    "itk_attention_batch": (C.c_int, [_vp, _u32, _u32, _u32p, _u64p, _u32, _vp, _vp, _vp, _vp]),
    "itk_attention_layers_host": (C.c_int, [_vp, _u32, _u32p, _u64p, _u32, _vp, _vp, _vp, _vp]),
    "itk_attention_batch_device": (C.c_int, [_vp, _u32, _u32, _u32p, _u64p, _u32, _vp, _vp, _vp, _vp]),
    "itk_layer_prep_set": (C.c_int, [_vp, _u32, C.POINTER(PrepConfig)]),
    "itk_attention_batch_prep": (C.c_int, [_vp, _u32, _u32, _u32p, _u64p, _u32, _vp, _vp, _vp, _vp]),
    "itk_attention_batch_prep_device": (C.c_int, [_vp, _u32, _u32, _u32p, _u64p, _u32, _vp, _vp, _vp, _vp]),
    "itk_decode_plan": (C.c_int, [_u32p, _u32, _u32, _u32, _u32, _u32p, _u32p]),
    "itk_decode_batch_limits": (C.c_int, [_u32, _u32, _u32p, _u32p, _u64p]),
    "itk_resident_begin": (C.c_int, [_vp, _u32, _u32p, _u64]),
    "itk_resident_layer": (C.c_int, [_vp, _u32, _vp, _vp, _vp, _vp]),
    "itk_resident_advance": (C.c_int, [_vp]),
    "itk_resident_end": (C.c_int, [_vp, _u64]),
    "itk_gather_create": (C.c_int, [_vp, _u32, _u32, _u64, C.POINTER(_vp), _vp]),
    "itk_gather_open": (C.c_int, [_vp, _u32, _vp]),
    "itk_gather_attach": (C.c_int, [_vp, _u32, _vp]),
    "itk_gather_close_peers": (C.c_int, [_vp]),
    "itk_gather_reset": (C.c_int, [_vp]),
    "itk_gather_status": (C.c_int, [_vp, _u32p]),
    "itk_resident_layer_gather": (C.c_int, [_vp, _u32, _vp, _vp, _vp, _u64]),
    "itk_gqa_attention": (C.c_int, [_vp, _u32, _u32, _vp, _sz, _u32, _u64p, _vp]),
    "itk_append": (C.c_int, [_vp, _u32, _u32, _vp, _sz, _vp, _sz, _u64]),
    "itk_append_rows": (C.c_int, [_vp, _u32, _u32, _vp, _vp, _u32, _u64]),
    "itk_append_rows_device": (C.c_int, [_vp, _u32, _u32, _u32p, _u64p, _u32, _vp, _vp]),
    "itk_profile_enable": (C.c_int, [_vp, _u32]),
    "itk_profile_read_copy": (C.c_int, [_vp, C.POINTER(C.c_double), _u64p]),
    "itk_profile_read": (C.c_int, [_vp, C.POINTER(C.c_double), _u64p, C.POINTER(C.c_double), _u64p]),
    "itk_next_position": (C.c_int, [_vp, _u32, _u32, _u64p]),
    "itk_stored_len": (C.c_int, [_vp, _u32, _u32, _u64p]),
    "itk_view_gather": (C.c_int, [_vp, _u32, _u32, _vp, _vp, _u64p, _u64p]),
    "itk_restore_bulk": (C.c_int, [_vp, _u32, _u32, _u64, _vp, _sz, _vp, _sz]),
    "itk_reset": (C.c_int, [_vp, _u32]),
    "itk_cache_checkpoint": (C.c_int, [_vp, _u32, _u64, C.POINTER(Checkpoint)]),
    "itk_cache_rewind": (C.c_int, [_vp, _u32, C.POINTER(Checkpoint), _u64]),
    "itk_cache_release": (C.c_int, [_vp, _u32, C.POINTER(Checkpoint)]),
    "itk_snapshot_capture": (C.c_int, [_vp, _u32, C.POINTER(_vp)]),
    "itk_snapshot_restore": (C.c_int, [_vp, _u32, _vp]),
    "itk_snapshot_free": (None, [_vp]),
    "itk_snapshot_token_count": (_u64, [_vp]),
    "itk_snapshot_payload_bytes": (_u64, [_vp]),
    "itk_snapshot_layer_to_host": (C.c_int, [_vp, _vp, _u32, _vp, _vp, _u64p, _u64p]),
    "itk_snapshot_from_host_f32": (C.c_int, [_vp, _u64, _u64p, _u64p, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp)]),
    "itk_snapshot_to_itkv": (C.c_int, [_vp, _vp, C.c_char_p, _vp, _sz, C.POINTER(_sz)]),
    "itk_snapshot_to_itkv_version": (C.c_int, [_vp, _vp, C.c_char_p, _u32, _vp, _sz, C.POINTER(_sz)]),
    "itk_snapshot_from_itkv": (C.c_int, [_vp, C.c_char_p, _sz, C.c_char_p, C.POINTER(_vp)]),
    "itk_itkv_check": (C.c_int, [C.c_char_p, _sz, _u32p, _u64p, _u32p, C.c_char_p, _sz]),
    "itk_draft_attention": (C.c_int, [_vp, _vp, _vp, _vp, _u32, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _u32, _u32, _u32,
                                      _u32, _u32, C.c_float, _vp, _vp, C.c_char_p, _sz]),
    "itk_prefix_store_open": (C.c_int, [C.c_char_p, _u64, C.POINTER(_vp)]),
    "itk_prefix_store_close": (None, [_vp]),
    "itk_prefix_store_last_error": (C.c_char_p, [_vp]),
    "itk_prefix_store_last_refusal": (C.c_char_p, [_vp]),
    "itk_prefix_store_rescan": (C.c_int, [_vp]),
    "itk_prefix_store_put": (C.c_int, [_vp, _u32p, _sz, _vp, _sz, _u64]),
    "itk_prefix_store_lookup": (C.c_int, [_vp, _u32p, _sz, C.POINTER(Config), C.c_char_p, _u64, _u64p, C.POINTER(_vp),
                                          C.POINTER(_sz)]),
    "itk_prefix_store_stats": (C.c_int, [_vp, _u64p, _u64p, _u64p]),
    "itk_prefix_store_entry": (C.c_int, [_vp, _u64, C.c_char_p, _sz, _u64p, _u64p, _u64p, _u64p, _u64p]),
    "itk_rope_rows": (C.c_int, [_vp, _vp, _u32, _u32, _u32, _u32, _u32, C.c_float, _vp, C.c_char_p, _sz]),
    "itk_decode_attention_noalloc": (C.c_int, [_vp, _vp, _u32, _u32, _u32, _u32, _u32, _u32p, _u32p, _vp, _vp, _u32, _vp,
                                               C.c_char_p, _sz]),
}

_lib = None


def load():
    """Load the shared library; raises (never falls back) when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise RuntimeError(
                f"{SO_PATH} is missing: build the sm_100a kernels first "
                "(python -m itak_torch_rebuild_b200.build, or __graft_entry__.build()); there is no CPU fallback"
            )
        lib = C.CDLL(SO_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
