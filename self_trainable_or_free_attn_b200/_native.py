"""ctypes binding of libechosparse_sm100.so (the C ABI declared in include/echosparse_sm100.h and
include/echosparse_vsa_sm100.h).

There is no fallback: if the library is missing or a call fails, this raises. PyTorch tensors are passed as raw device
pointers; the launch goes on torch's current CUDA stream.
"""
import ctypes
import functools
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# ECHOSPARSE_SM100_LIB selects another build of the same library (for example one compiled with other -D options).
LIB_PATH = os.environ.get("ECHOSPARSE_SM100_LIB") or os.path.join(_HERE, "_lib", "libechosparse_sm100.so")

_P = ctypes.c_void_p
_I = ctypes.c_int32
_F = ctypes.c_float
_I64 = ctypes.c_int64

# name -> argument types (all return int unless listed in _RESTYPES)
SIGNATURES = {
    "es_last_error": [],
    "es_abi_version": [],
    "es_launch_count": [],
    "es_device_status": [_P],
    "es_selftest_wait_timeout": [_I, _P],
    "es_exchange_rows": [_P, _I64, _I64, _P, _I64, _I64, _I, _I64, _I, _P],
    "es_block_attention": [_P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _F, _P],
    "es_sparse_attention": [_P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _F,
                            _P],
    "es_exact_fallback": [_P, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _P, _P],
    "es_compensate_fallback": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _P, _P],
    "es_block_means": [_P, _P, _P, _P, _I, _I, _P],
    "es_select_blocks": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P],
    "es_estimate_skipped": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _P],
    "es_full_step_scales": [_P, _P, _P, _P, _I, _I, _P],
    "es_pack_plan": [_P, _P, _I, _I, _I, _I, _P],
    "es_rebuild_plan": [_P, _P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _P],
    "es_reps_gram_splits": [_I],
    "es_reps_metric": [_P, _P, _P, _P, _P, _I, _I, _P],
    "es_reps_kmeans": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "es_reps_metric_static": [_P, _P, _P, _P, _I, _I, _P],
    "es_reps_metric_static_max_heads": [],
    "es_vsa_pool": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "es_vsa_router_lse": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "es_vsa_router_scores": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "es_vsa_topk_workspace_bytes": [_I, _I],
    "es_vsa_global_topk": [_P, _I, _I, _I, ctypes.c_longlong, _P, _P, _P, _P, _P, _P],
    "es_vsa_attn_fwd": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P],
    "es_vsa_attn_bwd_kv": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _P],
    "es_vsa_attn_bwd_q": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _P],
    "es_vsa_fuse_fwd": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "es_vsa_fuse_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "es_vsa_finalize": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "es_vsa_split_plan_workspace_bytes": [_I, _I],
    "es_vsa_split_plan": [_P, _I, _I, _I, _I, _I, ctypes.c_double, ctypes.c_double, _I, _I, _P, _P, _P, _P, _P],
    "es_vsa_attn_fwd_tasks": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _P],
    "es_vsa_split_merge_fwd": [_P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _P],
    "es_vsa_attn_bwd_kv_tasks": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _P, _P, _I, _I,
                                 _I, _I, _P],
    "es_vsa_attn_bwd_q_tasks": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _P],
    "es_vsa_split_merge_sum": [_P, _P, _P, _I, _P, _I, _P, _P, _P, _I, _I, _I, _P],
    "es_vsa_topk_bits_offset": [_I, _I],
    "es_vsa_block_scores": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "es_vsa_row_topk": [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _I, _P],
    "es_vsa_tier_attn_fwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "es_vsa_tier_attn_bwd_q": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I,
                               _I, _I, _I, _P],
    "es_vsa_tier_rep_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "es_vsa_tier_unpool": [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
}
_RESTYPES = {"es_last_error": ctypes.c_char_p, "es_launch_count": ctypes.c_longlong,
             "es_vsa_topk_workspace_bytes": ctypes.c_longlong, "es_vsa_split_plan_workspace_bytes": ctypes.c_longlong,
             "es_vsa_topk_bits_offset": ctypes.c_longlong}

_lib = None


class NativeError(RuntimeError):
    pass


def load():
    """Opens the shared library and declares every entry point. Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NativeError(f"{LIB_PATH} is missing: build it with `python -m self_trainable_or_free_attn_b200.build` "
                              f"(there is no CPU or Triton fallback)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = _RESTYPES.get(name, ctypes.c_int)
        _lib = lib
    return _lib


def last_error():
    return load().es_last_error().decode()


def check(status, what):
    if status != 0:
        raise NativeError(f"{what} failed ({status}): {last_error()}")


def device_status():
    """Synchronises the current device and returns (and clears) the kernels' status word; 0 means fine."""
    out = ctypes.c_int32(0)
    check(load().es_device_status(ctypes.byref(out)), "es_device_status")
    return out.value


def launch_count():
    return int(load().es_launch_count())


def device_guard(fn):
    """Decorator: runs `fn` with the CUDA device of its first tensor argument current, so that the stream looked up by
    `stream_ptr` and the launch itself follow the tensors and not whatever device the caller's thread had selected
    (reference: the OptionalCUDAGuard of csrc/vsa/vsa2_api.cpp:64, 80)."""
    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        import torch
        for a in args:
            if isinstance(a, torch.Tensor):
                if a.is_cuda and a.device.index != torch.cuda.current_device():
                    with torch.cuda.device(a.device):
                        return fn(*args, **kwargs)
                break
        return fn(*args, **kwargs)
    return wrapper


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def stream_ptr():
    import torch
    return torch.cuda.current_stream().cuda_stream
