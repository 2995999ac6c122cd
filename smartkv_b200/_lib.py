"""ctypes binding of libsmartkv_b200.so (the C ABI declared in include/smartkv_b200.h).

There is no fallback: if the library is missing the import of any operator fails
with an error that says how to build it.
"""
import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
# SMARTKV_B200_LIB points the loader at another build of the same ABI (e.g. an instrumented one)
LIB_PATH = os.environ.get("SMARTKV_B200_LIB") or os.path.join(HERE, "libsmartkv_b200.so")

NUM_BUCKETS = 4
BUCKET_BITS = (2, 3, 4, 8)
BITS_TO_BUCKET = {2: 0, 3: 1, 4: 2, 8: 3}
DTYPE_F32, DTYPE_F16 = 0, 1
ATTN_DEPENDENT_LAUNCH = 1      # flags of skv_decode_attention_masked

SKV_OK = 0


class StoreDesc(Structure):
    _fields_ = [
        ("num_layers", c_int32), ("num_seqs", c_int32), ("num_kv_heads", c_int32), ("head_dim", c_int32),
        ("cap", c_int32 * NUM_BUCKETS),
        ("row_bytes", c_int32 * NUM_BUCKETS), ("bucket_base", c_int32 * NUM_BUCKETS),
        ("slots", c_int32), ("reserved_", c_int32),
        ("k_off", c_int64 * NUM_BUCKETS), ("v_off", c_int64 * NUM_BUCKETS), ("sc_off", c_int64 * NUM_BUCKETS),
        ("arena_bytes", c_int64), ("total_bytes", c_int64),
    ]


ALLOC_MAX_PROTECTED = 16


class AllocConfig(Structure):
    """SkvAllocConfig of include/smartkv_b200.h."""
    _fields_ = [
        ("num_heads", c_int32), ("head_dim", c_int32), ("num_bits", c_int32), ("bits", c_int32 * 4),
        ("util", c_double * 4), ("memory_budget", c_double), ("importance_floor", c_double),
        ("rank_threshold", c_double), ("high_fraction", c_double), ("high_boost", c_double),
        ("hysteresis_intervals", c_int32), ("min_high_tokens", c_int32), ("scale_bits", c_int32),
        ("use_packing", c_int32), ("critical_window", c_int32), ("num_protected", c_int32),
        ("protected_ids", c_int32 * ALLOC_MAX_PROTECTED),
    ]


class SmartKVLibraryError(RuntimeError):
    pass


_lib = None

_SIGNATURES = {
    "skv_status_string": (c_char_p, [c_int]),
    "skv_build_arch": (c_int, []),
    "skv_store_layout": (c_int, [POINTER(StoreDesc)]),
    "skv_quantize_per_head": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "skv_pack": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "skv_unpack": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "skv_quantize_pack_append": (c_int, [POINTER(StoreDesc), c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                         c_void_p, c_void_p, c_void_p, c_void_p]),
    "skv_step_plan": (c_int, [POINTER(StoreDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_void_p]),
    "skv_step_commit": (c_int, [POINTER(StoreDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "skv_export_rows": (c_int, [POINTER(StoreDesc), c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "skv_dequant_rows": (c_int, [POINTER(StoreDesc), c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                 c_void_p, c_void_p, c_void_p]),
    "skv_import_rows": (c_int, [POINTER(StoreDesc), c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "skv_prefill_attention": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                      POINTER(c_int64), POINTER(c_int64), POINTER(c_int64), c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p]),
    "skv_attn_num_ctas": (c_int, [c_int]),
    "skv_attn_partials_bytes": (c_int64, [POINTER(StoreDesc), c_int, c_int]),
    "skv_attn_plan_bytes": (c_int64, [POINTER(StoreDesc), c_int]),
    "skv_attn_partials_per_run": (c_int, [POINTER(StoreDesc), c_int]),
    "skv_post_attention": (c_int, [POINTER(StoreDesc), c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                   c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                   c_void_p, c_void_p, c_void_p, c_float, c_float, c_void_p, c_void_p, c_void_p,
                                   c_int, c_void_p, c_void_p]),
    "skv_attn_plan": (c_int, [POINTER(StoreDesc), c_void_p, c_int, c_void_p, c_void_p]),
    "skv_decode_attention": (c_int, [POINTER(StoreDesc), c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                     c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "skv_decode_attention_masked": (c_int, [POINTER(StoreDesc), c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                            c_void_p, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_void_p,
                                            c_void_p]),
    "skv_set_dependent_launch": (c_int, [c_int]),
    "skv_set_attention_path": (c_int, [c_int]),
    "skv_get_attention_path": (c_int, []),
    "skv_set_wait_limit": (c_int, [ctypes.c_uint]),
    "skv_decode_attention_static": (c_int, [POINTER(StoreDesc), c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                            c_int, c_void_p, c_void_p, POINTER(c_void_p), c_void_p]),
    "skv_lse_combine": (c_int, [POINTER(StoreDesc), c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p,
                                c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "skv_lse_combine_masked": (c_int, [POINTER(StoreDesc), c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p,
                                       c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "skv_alloc_workspace_bytes": (c_int64, [POINTER(StoreDesc)]),
    "skv_alloc_bits": (c_int, [POINTER(StoreDesc), POINTER(AllocConfig), c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "skv_repack_plan_workspace_bytes": (c_int64, [POINTER(StoreDesc)]),
    "skv_repack_plan": (c_int, [POINTER(StoreDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_void_p]),
    "skv_requant_staging_bytes": (c_int64, [POINTER(StoreDesc), c_int64, c_int]),
    "skv_requant_repack": (c_int, [POINTER(StoreDesc), c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_int64, c_void_p, c_void_p]),
    "skv_repack_meta_staging_bytes": (c_int64, [POINTER(StoreDesc), c_int64]),
    "skv_repack_meta": (c_int, [POINTER(StoreDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p,
                                c_void_p]),
    "skv_importance_update": (c_int, [POINTER(StoreDesc), c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float,
                                      c_float, c_void_p]),
    "skv_read_error_flag": (c_int, [c_void_p, POINTER(c_int32), c_void_p]),
}


def exported_symbols():
    """Names every entry point the header declares (used by the CPU-side load test)."""
    return sorted(_SIGNATURES)


def lib():
    """Load the shared library once; raise loudly when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise SmartKVLibraryError(
            f"{LIB_PATH} is missing: build it with `python -m smartkv_b200.build` "
            "(needs nvcc; there is no CPU fallback for the SmartKV kernels)")
    handle = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(handle, name)
        fn.restype = res
        fn.argtypes = args
    _lib = handle
    return _lib


def check(status, what=""):
    if status != SKV_OK:
        msg = lib().skv_status_string(int(status)).decode()
        raise SmartKVLibraryError(f"{what or 'smartkv_b200 call'} failed: {msg} ({status})")


def ptr(t):
    """Device (or host) address of a torch tensor / None."""
    return None if t is None else c_void_p(t.data_ptr())


def stream_ptr(device=None):
    import torch
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)
