"""ctypes binding of libinfllm_b200.so (the C ABI declared in include/infllm_b200.h).

The library is the product: there is no Python or CPU fallback.  If it has not been built
(`python -m infllm_b200.build`) importing this module raises ImportError.
"""
import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("INFLLM_B200_LIB", os.path.join(_HERE, "libinfllm_b200.so"))  # the override is for instrumented builds

OK, E_BADARG, E_CAPACITY, E_CUDA, E_TIMEOUT, E_UNSUPPORTED, E_NOMEM = 0, -1, -2, -3, -4, -5, -6
BF16, FP16 = 0, 1
CACHE_LRU, CACHE_LRU_S = 0, 1
MASK_NONE, MASK_WINDOW, MASK_COMPLEMENT = 0, 1, 2
MAX_SEGMENTS = 80
PROF_ATTN, PROF_COLSUM, PROF_DECODE, PROF_TOPK, PROF_SLOTS = 0, 1, 2, 3, 4


class InfLLMError(RuntimeError):
    """A call into libinfllm_b200 returned an error code."""

    def __init__(self, code, message):
        super().__init__(f"infllm_b200 error {code}: {message}")
        self.code = code


class InfLLMCapacityError(InfLLMError, AssertionError):
    """The cache cannot hold a retrieval (the reference asserts in CudaCache.alloc)."""


class Config(ctypes.Structure):
    _fields_ = [
        ("n_heads", c_int32), ("n_kv_heads", c_int32), ("head_dim", c_int32),
        ("n_init", c_int32), ("n_local", c_int32), ("block_size", c_int32), ("max_cached_block", c_int32),
        ("topk", c_int32), ("exc_block_size", c_int32), ("repr_topk", c_int32),
        ("cache_strategy", c_int32), ("dtype", c_int32),
        ("score_decay", c_double), ("rope_base", c_float), ("rope_scale", c_float),
        ("device", c_int32), ("shard_rank", c_int32), ("shard_world", c_int32),
        ("debug_flags", c_int32), ("look_depth", c_int32), ("chunk_topk_calc", c_int32), ("device_store_mb", c_int32),
        ("reserved", c_int32 * 2),
    ]


class CtxInfo(ctypes.Structure):
    _fields_ = [(n, c_int64) for n in (
        "length", "frontier", "num_blocks", "init_len", "num_cached", "load_count", "exec_blocks",
        "h2d_bytes", "d2h_bytes", "cache_hits", "cache_misses", "evictions", "h2d_late_bytes", "inplace_units")]


class ShardCache(ctypes.Structure):
    """infllm_shard_cache of include/infllm_b200.h."""
    _fields_ = [
        ("lru", c_void_p), ("slot_of", c_void_p), ("free_slots", c_void_p),
        ("n_free", c_int32), ("id_lo", c_int32), ("n_owned", c_int32), ("pad", c_int32),
        ("load_count", c_int64), ("hits", c_int64), ("misses", c_int64),
        ("d_cache", c_void_p), ("h_units", c_void_p), ("unit_bytes", c_int64),
        ("d_slot_table", c_void_p), ("d_ptr_table", c_void_p),
    ]


# name -> (restype, argtypes); every symbol the header declares
class ShardToken(ctypes.Structure):
    """infllm_shard_token of include/infllm_b200.h."""
    _fields_ = [
        ("d_q", c_void_p), ("d_k", c_void_p), ("d_vin", c_void_p),
        ("q_hs", c_int64), ("k_hs", c_int64), ("v_hs", c_int64),
        ("d_q_loc", c_void_p), ("d_q_glb", c_void_p), ("d_qbar", c_void_p),
        ("d_k_raw", c_void_p), ("d_k_rot", c_void_p), ("d_v", c_void_p), ("d_score", c_void_p),
        ("d_cos", c_void_p), ("d_sin", c_void_p),
        ("cap", c_int64), ("at", c_int64),
        ("n_heads", c_int32), ("n_kv_heads", c_int32), ("head_dim", c_int32), ("dtype", c_int32), ("n_local", c_int32),
        ("block_size", c_int32), ("topk", c_int32), ("pad0", c_int32),
        ("d_block_k", c_void_p), ("d_scores", c_void_p),
        ("n_owned", c_int32), ("id_lo", c_int32),
        ("d_cand", c_void_p), ("d_status", c_void_p), ("h_status", c_void_p), ("d_slot_table", c_void_p),
        ("d_cache", c_void_p), ("unit_bytes", c_int64),
        ("share_at", c_int64), ("share_len", c_int64),
        ("d_init_k", c_void_p), ("d_init_v", c_void_p),
        ("ovf_at", c_int64), ("ovf_len", c_int64),
        ("init_len", c_int32), ("max_parts", c_int32),
        ("d_part_o", c_void_p), ("d_part_lse", c_void_p), ("d_logits", c_void_p),
        ("d_pack", c_void_p), ("d_out", c_void_p), ("d_lse", c_void_p),
        ("cand_off", c_int64), ("cand_slot", c_int64), ("cand_bytes", c_int64), ("part_off", c_int64),
        ("part_slot", c_int64), ("part_bytes", c_int64), ("flag1_off", c_int64), ("flag2_off", c_int64),
        ("seq", ctypes.c_uint32), ("wait_us", c_int32),
        ("d_unit_ptrs", c_void_p), ("d_ticket", c_void_p), ("ll_part_off", c_int64), ("ll_part_slot", c_int64), ("ll_cand_off", c_int64), ("ll_cand_slot", c_int64),
        ("d_stamps", c_void_p),
    ]


SIGNATURES = {
    "infllm_last_error": (c_char_p, []),
    "infllm_version": (c_char_p, []),
    "infllm_rope_table": (c_int, [POINTER(c_float), c_float, c_int, c_int64, c_void_p, c_void_p, c_void_p]),
    "infllm_rope_apply": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int, c_int64, c_int,
                                  c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p]),
    "infllm_attn_stage": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64,
                                  c_int, c_int, c_int64, c_int64, c_int, c_int, c_int64, c_int64,
                                  c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "infllm_attn_finalize": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p,
                                     c_int, c_int64, c_int, c_int, c_void_p]),
    "infllm_attn_colsum": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int, c_int, c_int64,
                                   c_int64, c_int, c_int, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int,
                                   c_int, c_void_p]),
    "infllm_block_topk": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                  c_int, c_void_p]),
    "infllm_block_score_rows": (c_int, [c_void_p, POINTER(c_int32), c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "infllm_repr_select": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int, c_int, c_int,
                                   c_int, c_int, c_int, c_void_p, c_int, c_void_p]),
    "infllm_attn_decode_max_parts": (c_int64, [c_int, c_int64]),
    "infllm_attn_decode": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, POINTER(c_void_p),
                                   POINTER(c_void_p), POINTER(c_int64), POINTER(c_int32), POINTER(c_int32),
                                   c_void_p, c_void_p, c_int, POINTER(c_int), c_int, c_void_p, c_int, c_void_p]),
    "infllm_attn_decode_noalloc": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, POINTER(c_void_p),
                                           POINTER(c_void_p), POINTER(c_int64), POINTER(c_int32), POINTER(c_int32),
                                           c_void_p, c_int64, c_void_p, c_int, c_void_p]),
    "infllm_lse_merge": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int64, c_void_p, c_int,
                                 c_void_p]),
    "infllm_lse_merge_ex": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_int64, c_void_p,
                                    c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p]),
    "infllm_attn_decode_units": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, POINTER(c_void_p),
                                         POINTER(c_void_p), POINTER(c_int64), POINTER(c_int32), POINTER(c_int32),
                                         c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int64, c_void_p,
                                         c_void_p, c_void_p, c_int, POINTER(c_int), c_int, c_void_p, c_int, c_void_p]),
    "infllm_slot_table_update": (c_int, [c_void_p, POINTER(c_int32), POINTER(c_int32), c_int, c_void_p]),
    "infllm_shard_refill": (c_int, [POINTER(ShardCache), c_void_p, c_int, c_void_p]),
    "infllm_ptr_table_update": (c_int, [c_void_p, POINTER(c_int32), POINTER(ctypes.c_uint64), c_int, c_void_p]),
    "infllm_mailbox_handle_bytes": (c_int, []),
    "infllm_mailbox_create": (c_int, [c_int64, c_int, c_int, c_void_p, POINTER(c_void_p)]),
    "infllm_mailbox_open": (c_int, [c_void_p, c_void_p]),
    "infllm_mailbox_alias": (c_int, [c_void_p, c_int, c_void_p]),
    "infllm_mailbox_local": (c_void_p, [c_void_p]),
    "infllm_mailbox_destroy": (c_int, [c_void_p]),
    "infllm_mailbox_put": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, ctypes.c_uint32, c_void_p]),
    "infllm_mailbox_wait": (c_int, [c_void_p, c_int64, ctypes.c_uint32, c_int, c_void_p, c_int64, c_int64, c_int64,
                                    c_void_p, c_void_p, c_void_p]),
    "infllm_topk_pairs": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "infllm_shard_token_run": (c_int, [POINTER(ShardToken), c_void_p, c_void_p]),
    "infllm_ingest_token": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64,
                                    c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int,
                                    c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "infllm_unit_fetch": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "infllm_comm_id_bytes": (c_int, []),
    "infllm_comm_unique_id": (c_int, [c_void_p]),
    "infllm_comm_create": (c_int, [c_void_p, c_int, c_int, POINTER(c_void_p)]),
    "infllm_comm_destroy": (c_int, [c_void_p]),
    "infllm_ctx_set_comm": (c_int, [c_void_p, c_void_p]),
    "infllm_ctx_save": (c_int, [c_void_p, c_char_p, c_void_p]),
    "infllm_ctx_load": (c_int, [c_void_p, c_char_p, c_void_p]),
    "infllm_ctx_create": (c_int, [POINTER(Config), POINTER(c_void_p)]),
    "infllm_ctx_destroy": (c_int, [c_void_p]),
    "infllm_ctx_reset": (c_int, [c_void_p]),
    "infllm_ctx_append": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p,
                                  c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "infllm_ctx_get_info": (c_int, [c_void_p, POINTER(CtxInfo)]),
    "infllm_ctx_profile": (c_int, [c_void_p, c_int]),
    "infllm_ctx_get_profile": (c_int, [c_void_p, POINTER(c_double), POINTER(c_double), POINTER(c_int64)]),
    "infllm_device_error": (c_int, [POINTER(c_int), POINTER(c_int)]),
    "infllm_device_error_set": (c_int, [c_int, c_int]),
    "infllm_device_store_reserve": (c_int, [c_int, c_int64]),
    "infllm_device_store_release": (c_int, [c_int]),
    "infllm_device_store_info": (c_int, [c_int, POINTER(c_int64), POINTER(c_int64)]),
    "infllm_launch_count": (ctypes.c_longlong, []),
    "infllm_ctx_trace": (c_int, [c_void_p, c_int]),
    "infllm_ctx_get_trace": (c_int, [c_void_p, POINTER(c_int32), POINTER(c_int64), POINTER(c_float), c_int, POINTER(c_int)]),
    "infllm_ctx_get_host_timers": (c_int, [c_void_p, POINTER(c_double)]),
    "infllm_ctx_get_cached": (c_int, [c_void_p, POINTER(c_int32), POINTER(c_double), c_int, POINTER(c_int)]),
    "infllm_ctx_get_topk": (c_int, [c_void_p, c_int64, POINTER(c_int32), c_int, POINTER(c_int)]),
    "infllm_ctx_get_block_k": (c_int, [c_void_p, c_int64, c_int64, c_void_p]),
    "infllm_ctx_load_synthetic": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p]),
    "infllm_lru_create": (c_int, [c_int, POINTER(c_void_p)]),
    "infllm_lru_destroy": (c_int, [c_void_p]),
    "infllm_lru_plan": (c_int, [c_void_p, POINTER(c_int32), c_int, POINTER(c_int32), POINTER(c_int)]),
    "infllm_lru_stamp": (c_int, [c_void_p, POINTER(c_int32), c_int, c_double]),
    "infllm_lru_scale": (c_int, [c_void_p, c_double]),
    "infllm_lru_add": (c_int, [c_void_p, c_int32, c_double]),
    "infllm_lru_items": (c_int, [c_void_p, POINTER(c_int32), POINTER(c_double), c_int, POINTER(c_int)]),
}

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build the CUDA library first (python -m infllm_b200.build). "
        "infllm_b200 has no fallback implementation.")

lib = ctypes.CDLL(LIB_PATH)
for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError here means the library is stale
    _fn.restype = _res
    _fn.argtypes = _args


def check(rc):
    """Raise for a non-zero return code of the C ABI."""
    if rc == OK:
        return
    msg = lib.infllm_last_error().decode("utf-8", "replace")
    if rc == E_CAPACITY:
        raise InfLLMCapacityError(rc, msg)
    raise InfLLMError(rc, msg)


def dtype_code(dtype):
    import torch

    if dtype == torch.bfloat16:
        return BF16
    if dtype == torch.float16:
        return FP16
    raise TypeError(f"infllm_b200 kernels take bfloat16 or float16 activations, got {dtype}")


def stream_ptr(device=None):
    import torch

    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(t, what):
    if not t.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA tensor: infllm_b200 has no CPU path")


def device_error():
    """(code, where) of the tensor-core kernels' error record; clears it.  Synchronises the device."""
    code, where = c_int(), c_int()
    check(lib.infllm_device_error(ctypes.byref(code), ctypes.byref(where)))
    return code.value, where.value
