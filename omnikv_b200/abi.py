"""ctypes binding of ``libomnikv_b200.so`` (the C ABI declared in ``include/omnikv_b200.h``).

There is no fallback: if the library is missing, ``lib()`` raises with the build command.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

# OMNIKV_B200_LIB selects another build of the same library (the profiling build of ``build.py --trace``)
_LIB_PATH = Path(os.environ.get("OMNIKV_B200_LIB") or Path(__file__).resolve().parent / "_lib" / "libomnikv_b200.so")
_lib = None

ABI_VERSION = 5
F32, BF16, F16 = 0, 1, 2
SEL_SOFTMAX_LAST, SEL_UNIFORM, SEL_EXP = 0, 1, 2
NO_ALLOC_SCRATCH_BYTES = 4 * 1024 * 1024

c_i32p = C.POINTER(C.c_int32)
c_f32p = C.POINTER(C.c_float)


class AttnParams(C.Structure):
    """Mirror of ``omnikv_attn_params``."""

    _fields_ = [
        ("dtype", C.c_int32), ("B", C.c_int32), ("H", C.c_int32), ("KVH", C.c_int32), ("head_dim", C.c_int32),
        ("scale", C.c_float),
        ("q", C.c_void_p), ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64),
        ("out", C.c_void_p),
        ("kA", C.c_void_p), ("vA", C.c_void_p),
        ("a_stride_b", C.c_int64), ("a_stride_h", C.c_int64), ("a_stride_row", C.c_int64),
        ("idxA", C.c_void_p), ("idx_stride", C.c_int64), ("idx_row", C.c_void_p), ("lenA", C.c_void_p),
        ("kB", C.c_void_p), ("vB", C.c_void_p),
        ("b_stride_b", C.c_int64), ("b_stride_h", C.c_int64), ("b_stride_row", C.c_int64),
        ("startB", C.c_void_p), ("lenB", C.c_void_p),
        ("score_out", C.c_void_p), ("score_stride", C.c_int64), ("score_len", C.c_void_p),
        ("n_splits", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("status", C.c_void_p), ("a_rows", C.c_int64),
    ]


class WindowParams(C.Structure):
    """Mirror of ``omnikv_window_params``."""

    _fields_ = [
        ("dtype", C.c_int32), ("B", C.c_int32), ("H", C.c_int32), ("KVH", C.c_int32), ("head_dim", C.c_int32),
        ("W", C.c_int32), ("selector", C.c_int32), ("scale", C.c_float),
        ("qw", C.c_void_p), ("k", C.c_void_p),
        ("k_stride_b", C.c_int64), ("k_stride_h", C.c_int64), ("k_stride_row", C.c_int64),
        ("consider_len", C.c_void_p), ("max_len", C.c_int32),
        ("score_out", C.c_void_p), ("planes_out", C.c_void_p), ("score_stride", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("status", C.c_void_p),
    ]


class PrefillParams(C.Structure):
    """Mirror of ``omnikv_prefill_params``."""

    _fields_ = [
        ("dtype", C.c_int32), ("B", C.c_int32), ("H", C.c_int32), ("KVH", C.c_int32), ("head_dim", C.c_int32),
        ("Sq", C.c_int32), ("Skv", C.c_int32), ("q_pos0", C.c_int32), ("scale", C.c_float),
        ("q", C.c_void_p), ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64), ("q_stride_row", C.c_int64),
        ("k", C.c_void_p), ("k_stride_b", C.c_int64), ("k_stride_h", C.c_int64), ("k_stride_row", C.c_int64),
        ("v", C.c_void_p), ("v_stride_b", C.c_int64), ("v_stride_h", C.c_int64), ("v_stride_row", C.c_int64),
        ("out", C.c_void_p), ("o_stride_b", C.c_int64), ("o_stride_row", C.c_int64), ("o_stride_h", C.c_int64),
        ("status", C.c_void_p), ("variant", C.c_int32),
    ]


class BatchedLinearParams(C.Structure):
    """Mirror of ``omnikv_batched_linear_params``."""

    _fields_ = [
        ("dtype", C.c_int32), ("n_tokens", C.c_int32), ("w_rows", C.c_int32), ("K", C.c_int32),
        ("w", C.c_void_p), ("w_stride_row", C.c_int64), ("x", C.c_void_p), ("x_stride_tok", C.c_int64),
        ("norm_w", C.c_void_p), ("eps", C.c_float), ("epilogue", C.c_int32),
        ("residual", C.c_void_p), ("residual_stride_tok", C.c_int64), ("out", C.c_void_p),
        ("out_stride_tok", C.c_int64), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("status", C.c_void_p),
    ]


EPI_STORE, EPI_STORE_F32, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2, 3


class TpExchange(C.Structure):
    """Mirror of ``omnikv_tp_exchange``."""

    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("peer_base", C.c_void_p * 8),
                ("done_counter", C.c_void_p), ("epoch", C.c_void_p), ("seq", C.c_int32), ("hidden", C.c_int32)]


class ChainParams(C.Structure):
    """Mirror of ``omnikv_chain_params``."""

    _fields_ = [
        ("dtype", C.c_int32), ("hidden", C.c_int32), ("inter", C.c_int32), ("H", C.c_int32), ("KVH", C.c_int32),
        ("eps", C.c_float),
        ("h", C.c_void_p), ("w_o", C.c_void_p), ("attn_out", C.c_void_p), ("post_norm_w", C.c_void_p),
        ("w_gate_up", C.c_void_p), ("w_down", C.c_void_p), ("act_scratch", C.c_void_p),
        ("in_norm_w", C.c_void_p), ("w_qkv", C.c_void_p), ("inv_freq", C.c_void_p), ("rope_pos", C.c_void_p),
        ("q_out", C.c_void_p), ("k_cache_seq", C.c_void_p), ("v_cache_seq", C.c_void_p),
        ("kv_stride_h", C.c_int64), ("kv_stride_row", C.c_int64), ("cache_pos", C.c_void_p),
        ("final_norm_w", C.c_void_p), ("w_head", C.c_void_p), ("vocab_rows", C.c_int32),
        ("logits", C.c_void_p), ("best_scratch", C.c_void_p), ("token_out", C.c_void_p),
        ("grid_sync", C.c_void_p), ("chunk_counters", C.c_void_p), ("status", C.c_void_p),
        ("next_w", C.c_void_p), ("next_w_bytes", C.c_size_t),
    ]


# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "omnikv_abi_version": (C.c_int, []),
    "omnikv_strerror": (C.c_char_p, [C.c_int]),
    "omnikv_last_cuda_error": (C.c_char_p, []),
    "omnikv_decode_attn_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "omnikv_decode_attn": (C.c_int, [C.POINTER(AttnParams), C.c_void_p]),
    "omnikv_decode_attn_no_alloc": (C.c_int, [C.POINTER(AttnParams), C.c_void_p]),
    "omnikv_score_window_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "omnikv_score_window": (C.c_int, [C.POINTER(WindowParams), C.c_void_p]),
    "omnikv_prefill_attn": (C.c_int, [C.POINTER(PrefillParams), C.c_void_p]),
    "omnikv_batched_linear_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "omnikv_batched_linear": (C.c_int, [C.POINTER(BatchedLinearParams), C.c_void_p]),
    "omnikv_window_fold": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_void_p, C.c_int,
                                     C.c_int, C.c_void_p]),
    "omnikv_topk_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "omnikv_topk": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p,
                              C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_size_t,
                              C.c_void_p]),
    "omnikv_offload_gather": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                        C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "omnikv_tp_exchange_bytes": (C.c_size_t, [C.c_int]),
    "omnikv_decode_qkv": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                    C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                    C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "omnikv_decode_gemv_residual": (C.c_int, [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                              C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "omnikv_decode_gate_up": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_int, C.c_int,
                                        C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "omnikv_decode_logits": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_int, C.c_int,
                                       C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_void_p]),
    "omnikv_decode_chain": (C.c_int, [C.POINTER(ChainParams), C.c_void_p]),
    "omnikv_decode_chain_supported": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "omnikv_idx_commit": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int,
                                    C.c_int, C.c_double, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "omnikv_tp_allreduce_sum": (C.c_int, [C.c_int, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "omnikv_tp_allreduce_max": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "omnikv_tp_allgather": (C.c_int, [C.c_int, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "omnikv_rope_append": (C.c_int, [C.c_int, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                     C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                     C.c_int64, C.c_void_p, C.c_void_p]),
    "omnikv_add_rms_norm": (C.c_int, [C.c_int, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_float,
                                      C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "omnikv_rope_window": (C.c_int, [C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int,
                                     C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "omnikv_silu_mul": (C.c_int, [C.c_int, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "omnikv_kv_append": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                   C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
                                   C.c_void_p]),
}


def lib_path() -> Path:
    return _LIB_PATH


def lib():
    """The loaded library.  Raises when it has not been built: there is no other code path."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: build it with `python -m omnikv_b200.build` (needs nvcc). "
                "omnikv_b200 has no CPU or PyTorch fallback for its kernels."
            )
        handle = C.CDLL(str(_LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is not exported
            fn.restype, fn.argtypes = res, args
        got = handle.omnikv_abi_version()
        if got != ABI_VERSION:
            raise RuntimeError(f"libomnikv_b200 ABI {got} != binding ABI {ABI_VERSION}: rebuild the library")
        _lib = handle
    return _lib


class OmniKVError(RuntimeError):
    pass


def check(status: int, what: str) -> None:
    if status != 0:
        l = lib()
        msg = l.omnikv_strerror(status).decode()
        extra = l.omnikv_last_cuda_error().decode() if status == -4 else ""
        raise OmniKVError(f"{what}: {msg}{(' -- ' + extra) if extra else ''}")
