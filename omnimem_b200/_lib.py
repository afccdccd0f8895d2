"""ctypes binding of libomnimem_b200.so (the C ABI declared in include/omnimem_b200.h).

The library is the only compute path of this package: if it is missing, loading raises -
there is no Python or CPU stand-in.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libomnimem_b200.so")

NSA_BF16, NSA_F16, NSA_F32 = 0, 1, 2
NSA_KV_DENSE, NSA_KV_PAGED, NSA_KV_PTR = 0, 1, 2
NSA_ERR_EXHAUSTED = -6


class NSABackendError(RuntimeError):
    """A call into the CUDA library failed (mirrors the reference's NSABackendError,
    nsa/cuda_backend/ops.py:16-24)."""


class KVSource(C.Structure):
    _fields_ = [
        ("mode", C.c_int32), ("k", C.c_void_p), ("v", C.c_void_p),
        ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3), ("n_tokens", C.c_int64),
        ("block_table", C.c_void_p), ("max_blocks", C.c_int32), ("page_tokens", C.c_int32),
        ("ptr_k", C.c_void_p), ("ptr_v", C.c_void_p), ("ptr_stride_n", C.c_int64), ("num_pages", C.c_int64),
    ]


class Rope(C.Structure):
    """nsa_rope: three complex128 frequency tables and the chunk's grid / token order."""
    _fields_ = [("freqs_f", C.c_void_p), ("freqs_h", C.c_void_p), ("freqs_w", C.c_void_p)] + [
        (n, C.c_int32) for n in ("c_f", "c_h", "c_w", "grid_h", "grid_w", "pool_f", "pool_h", "pool_w", "start_frame")]


class TopkMask(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "block_size", "chunk_size", "chunk_size_k", "q_group_size", "q_chunk_offset", "ex_win",
        "ex_sink", "causal", "tf_mask", "prog_excl", "id_base", "id_stride")]


_i32, _i64, _f32, _vp, _sz = C.c_int32, C.c_int64, C.c_float, C.c_void_p, C.c_size_t
_S3 = C.POINTER(C.c_int64)

# name -> (restype, argtypes); must list every function declared in include/omnimem_b200.h
PROTOTYPES = {
    "nsa_last_error": (C.c_char_p, []),
    "nsa_version": (C.c_char_p, []),
    "nsa_device_status": (_i32, [C.POINTER(C.c_int32)]),
    "nsa_pool_rows": (_i32, [_vp, _S3, _vp, _S3, _i32, _i64, _i32, _i32, _i32, _i32, _vp]),
    "nsa_topk_workspace_bytes": (_sz, [_i32, _i32, _i32, _i64]),
    "nsa_topk": (_i32, [_vp, _S3, _vp, _S3, _i32, _i32, _i32, _i32, _i64, _i32, _f32,
                        C.POINTER(TopkMask), _vp, _vp, _vp, _sz, _i32, _vp]),
    "nsa_topk_static_scratch_max_scores": (_sz, []),
    "nsa_topk_static_scratch": (_i32, [_vp, _S3, _vp, _S3, _i32, _i32, _i32, _i32, _i64, _i32, _f32,
                                       C.POINTER(TopkMask), _vp, _vp, _i32, _vp]),
    "nsa_pool_score_topk": (_i32, [_vp, _S3, _vp, _S3, _i32, _i32, _i32, _i32, _i64, _i32, _f32,
                                   C.POINTER(TopkMask), _vp, _vp, _vp, _vp, _sz, _i32, _vp]),
    "nsa_select_blocks": (_i32, [_vp, _S3, _vp, _S3, _i32, _i64, _i32, _i32, _i64, _i32, _f32,
                                 C.POINTER(TopkMask), _vp, _vp, _vp, _vp, _vp, _sz, _i32, _vp]),
    "nsa_merge_candidates": (_i32, [_vp, _vp, _i32, _i64, _i32, _i32, _vp, _vp, _vp]),
    "nsa_sel_fwd": (_i32, [_vp, _S3, C.POINTER(KVSource), _vp, _S3, _vp, _S3, _vp, _i32, _i64, _i32,
                           _i32, _i32, _i32, _i32, _i32, _i32, _f32, _i32, _vp]),
    "nsa_probe_bulk_stream": (_i32, [_vp, _sz, _i32, _vp]),
    "nsa_range_fwd_workspace_bytes": (_sz, [_i32, _i64, _i32, _i32, _i32]),
    "nsa_range_fwd": (_i32, [_vp, _S3, C.POINTER(KVSource), _i32, _i32, _vp, _S3, _vp, _i32, _i64, _i32, _i32,
                             _i32, _f32, _vp, _sz, _i32, _vp]),
    "nsa_inverted_index_workspace_bytes": (_sz, [_i32, _i32, _i64]),
    "nsa_inverted_index": (_i32, [_vp, _S3, _i32, _i32, _i32, _i32, _i64, _i32, _i32, _i32, _i32,
                                  _vp, _vp, _vp, _sz, _vp]),
    "nsa_sel_bwd_workspace_bytes": (_sz, [_i32, _i64, _i32, _i64, _i32, _i32, _i32]),
    "nsa_sel_bwd": (_i32, [_vp, _S3, C.POINTER(KVSource), _vp, _S3, _vp, _S3, _vp, _vp, _S3, _vp, _S3,
                           _vp, _vp, _i32, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32,
                           _vp, _sz, _i32, _vp]),
    "nsa_sel_bwd_dq": (_i32, [_vp, _S3, C.POINTER(KVSource), _vp, _S3, _vp, _S3, _vp, _vp, _S3, _vp, _S3, _vp,
                              _i32, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _i32, _vp]),
    "nsa_sel_bwd_dkv": (_i32, [_vp, _S3, C.POINTER(KVSource), _vp, _vp, _vp, _vp, _vp, _S3, _vp, _vp,
                               _i32, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _vp, _sz, _i32, _vp]),
    "nsa_sel_bwd_pds_bytes": (_sz, [_i32, _i64, _i32, _i32, _i32]),
    "nsa_inverted_index_slots": (_i32, [_vp, _S3, _i32, _i32, _i32, _i32, _i64, _i32, _i32, _i32, _i32,
                                        _vp, _vp, _vp, _vp, _sz, _vp]),
    "nsa_sel_bwd_dq_pds": (_i32, [_vp, _S3, C.POINTER(KVSource), _vp, _S3, _vp, _S3, _vp, _vp, _S3, _vp, _S3, _vp,
                                  _i32, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _vp, _sz,
                                  C.POINTER(C.c_int32), _i32, _vp]),
    "nsa_sel_bwd_dkv_pds": (_i32, [_vp, _S3, C.POINTER(KVSource), _vp, _vp, _vp, _vp, _sz, _vp, _vp, _vp, _S3, _vp, _vp,
                                   _i32, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _vp, _sz, _i32, _vp]),
    "nsa_local_block_ids": (_i32, [_vp, _i64, _i32, _i32, _vp, _vp]),
    "nsa_merge_partials": (_i32, [_vp, _vp, _i32, _i32, _i64, _i32, _i32, _vp, _vp, _i32, _vp]),
    "nsa_merge_packed_rows": (_i32, [_vp, _i32, _i64, _i32, _i32, _vp, _i32, _vp]),
    "nsa_sel_bwd_dkv_ptr": (_i32, [_vp, _S3, _vp, _vp, _vp, _vp, _S3, _i32, _vp, _i64, _i64, _i64, _i64, _i32, _i64,
                                   _i64, _vp, _vp, _i64, _vp, _vp, _vp, _S3, _i32, _i64, _i32, _i32, _i32, _i32, _i32,
                                   _f32, _i32, _vp]),
    "nsa_gate_combine": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _vp]),
    "nsa_gate_combine_bwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _vp]),
    "nsa_build_ptr_table": (_i32, [_vp, _S3, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i64,
                                   _i32, _i64, _vp, _vp, _vp]),
    "nsa_cache_append": (_i32, [_vp, _vp, _S3, _i64, _i64, _i64, _i32, _i32, _vp, _vp, _i32, _vp, _i32,
                                _vp, _i32, _vp, _vp, _i64, _vp, _vp, _vp, _i32, _vp]),
    "nsa_cache_append_rope": (_i32, [_vp, _vp, _S3, _i64, _i64, _i64, _i32, _i32, _vp, _vp, _i32, _vp, _i32,
                                     _vp, _i32, _vp, _vp, _i64, _vp, _vp, _vp, _i32, C.POINTER(Rope), _vp]),
    "nsa_rope_apply": (_i32, [_vp, _S3, _i64, _i32, _i32, _vp, _i32, C.POINTER(Rope), _vp]),
    "nsa_cache_dedup_workspace_bytes": (_sz, [_i64]),
    "nsa_cache_dedup_touch": (_i32, [_vp, _i64, _i32, _i32, _i32, _i32, _vp, _i32, _vp, _vp, _i64,
                                     _vp, _vp, _i32, _vp, _vp, _sz, _vp]),
    "nsa_cache_select_victims": (_i32, [_vp, _vp, _i32, _i32, _i32, _i64, _i32, _vp, _i32, _vp, _vp, _vp]),
    "nsa_cache_move_pages": (_i32, [_i32, _vp, _vp, _i32, _vp, _i32, _vp, _vp, _i64, _vp, _vp, _vp,
                                    _vp, _vp, _i64, _vp, _vp]),
    "nsa_gather_publish_clear": (_i32, [_vp, _i64, _i64, _i64, _i32, _i32, C.POINTER(C.c_int64), _vp]),
    "nsa_block_range": (_i32, [_vp, _vp, _i32, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i32,
                               _i32, _i32, _vp]),
}

_lock = threading.Lock()
_lib = None


def load() -> C.CDLL:
    """Load the library once (thread safe) and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise NSABackendError(
                f"{LIB_PATH} is missing: build it with `python -m omnimem_b200.build` "
                "(nvcc, sm_100a). There is no fallback path.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def call(name: str, *args) -> None:
    """Call an int-returning entry point; a non-zero status raises NSABackendError with the
    library's message."""
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        msg = lib.nsa_last_error().decode("utf-8", "replace")
        raise NSABackendError(f"{name} failed ({rc}): {msg}")


def device_status() -> int:
    """Read and clear the device-side status word (synchronises)."""
    v = C.c_int32(0)
    call("nsa_device_status", C.byref(v))
    return int(v.value)


def strides3(t, dims=(0, 1, 2)):
    return (C.c_int64 * 3)(*[t.stride(d) for d in dims])


def strides4(t):
    return (C.c_int64 * 4)(*t.stride())
