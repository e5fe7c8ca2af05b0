"""ctypes bindings of include/bullet_b200.h.  There is no fallback: a missing library is an error."""
from __future__ import annotations

import ctypes
import os

from .configs import CNetDesc

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libbullet_b200.so")

#: every symbol the header declares; `load()` checks that the library exports each one
SYMBOLS = (
    "b200_last_error", "b200_version", "b200_net_create", "b200_net_destroy", "b200_net_set_option",
    "b200_net_tensor_size", "b200_net_set_tensor", "b200_net_get_tensor", "b200_net_set_adamw",
    "b200_batch_upload", "b200_step", "b200_backward", "b200_update", "b200_grad_buffer", "b200_loss",
    "b200_forward", "b200_sync", "b200_get_timings", "b200_net_get_activation", "b200_map_chess768",
    "b200_map_chess_buckets_mirrored", "b200_map_ataxx147", "b200_material_count", "b200_make_targets",
    "b200_pack_indices_u16", "b200_unpack_indices_u16", "b200_net_get_stat", "b200_op_ft_forward", "b200_op_ft_forward_noalloc",
    "b200_backward_begin", "b200_backward_ft", "b200_backward_end", "b200_grad_part", "b200_update_range",
    "b200_update_end", "b200_loss_of", "b200_checkpoint_save", "b200_checkpoint_load", "b200_flat_buffer",
    "b200_net_tensor_shape", "b200_quant_size", "b200_quantise", "b200_transpose", "b200_saved_format_size",
    "b200_saved_format_write", "b200_save_quantised", "b200_save_unquantised",
    "b200_forward_begin", "b200_forward_ft", "b200_net_tensor_offset",
    "b200_exchange_export", "b200_exchange_import", "b200_update_exchange", "b200_update_exchange_range",
    "b200_grad_zero_range", "b200_batch_upload_records", "b200_set_host_threads", "b200_step_exchange",
    "b200_batch_upload_records_gpu", "b200_slot_read", "b200_probe_bandwidth", "b200_net_set_optimiser",
)


class CAdamW(ctypes.Structure):
    _fields_ = [(n, ctypes.c_float) for n in ("decay", "beta1", "beta2", "min_weight", "max_weight")]


class COptimiser(ctypes.Structure):
    """b200_optimiser_params: kind 0 AdamW, 1 RAdam, 2 Ranger."""

    _fields_ = [("kind", ctypes.c_int32)] + [(n, ctypes.c_float) for n in ("decay", "beta1", "beta2", "min_weight", "max_weight",
                                                                         "n_sma_threshold", "alpha")] + [("k", ctypes.c_int32)]


class CFtOp(ctypes.Structure):
    """b200_ft_op: the operator-level feature-transformer forward on device pointers."""

    _fields_ = [(n, ctypes.c_int32) for n in ("n_inputs", "nnz", "ft_out", "ft_act", "pairwise", "ft_block_rows", "n")] + \
               [(n, ctypes.c_void_p) for n in ("table", "bias", "idx_stm", "idx_nstm", "x", "u")]


class CSavedFormat(ctypes.Structure):
    """b200_saved_format: one entry of an export (custom bytes, or a weight with transforms and a quantisation)."""

    _fields_ = [("id", ctypes.c_char_p), ("custom", ctypes.c_void_p), ("custom_len", ctypes.c_int64)] + \
               [(n, ctypes.c_int32) for n in ("quant", "multiplier", "round", "transpose", "merge_factoriser")]


class CTimings(ctypes.Structure):
    _fields_ = [(n, ctypes.c_float) for n in
                ("ft_forward", "dense_forward", "dense_backward", "ft_backward", "factoriser_grad", "optimiser",
                 "total")] + [("steps", ctypes.c_int32)]


class B200Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"bullet_b200 error {code}: {message}")
        self.code = code


_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m bullet_b200.build` (needs nvcc). "
            "bullet_b200 has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    missing = [s for s in SYMBOLS if not hasattr(lib, s)]
    if missing:
        raise ImportError(f"{LIB_PATH} does not export {missing}; rebuild it")
    vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_float
    cp = ctypes.c_char_p
    lib.b200_last_error.restype = cp
    sigs = {
        "b200_net_create": [ctypes.c_int, vp, ctypes.POINTER(CNetDesc), ctypes.POINTER(vp)],
        "b200_net_destroy": [vp],
        "b200_net_set_option": [vp, cp, i64],
        "b200_net_tensor_size": [vp, cp, ctypes.POINTER(i64)],
        "b200_net_set_tensor": [vp, cp, ctypes.c_int, vp, i64],
        "b200_net_get_tensor": [vp, cp, ctypes.c_int, vp, i64],
        "b200_net_set_adamw": [vp, cp, ctypes.POINTER(CAdamW)],
        "b200_net_set_optimiser": [vp, cp, ctypes.POINTER(COptimiser)],
        "b200_batch_upload": [vp, ctypes.c_int, vp, vp, vp, vp, i32],
        "b200_batch_upload_records": [vp, ctypes.c_int, vp, i32, i32, vp, f32, f32],
        "b200_batch_upload_records_gpu": [vp, ctypes.c_int, vp, i32, i32, vp, f32, f32],
        "b200_slot_read": [vp, ctypes.c_int, vp, vp, vp, vp, vp, vp, ctypes.POINTER(i32)],
        "b200_step": [vp, ctypes.c_int, f32, f32],
        "b200_backward": [vp, ctypes.c_int],
        "b200_update": [vp, f32, f32],
        "b200_forward_begin": [vp, ctypes.c_int],
        "b200_forward_ft": [vp, ctypes.c_int, ctypes.c_int, ctypes.c_int],
        "b200_net_tensor_offset": [vp, cp, ctypes.POINTER(i64)],
        "b200_exchange_export": [vp, vp, i64],
        "b200_exchange_import": [vp, ctypes.c_int, ctypes.c_int, vp, i64],
        "b200_update_exchange": [vp, f32, f32],
        "b200_step_exchange": [vp, ctypes.c_int, f32, f32],
        "b200_update_exchange_range": [vp, f32, f32, i64, i64, ctypes.c_int, vp],
        "b200_grad_zero_range": [vp, i64, i64],
        "b200_backward_begin": [vp, ctypes.c_int],
        "b200_backward_ft": [vp, ctypes.c_int, ctypes.c_int, ctypes.c_int],
        "b200_backward_end": [vp, ctypes.c_int],
        "b200_grad_part": [vp, ctypes.c_int, ctypes.c_int, ctypes.POINTER(i64), ctypes.POINTER(i64)],
        "b200_update_range": [vp, f32, f32, i64, i64],
        "b200_update_end": [vp],
        "b200_grad_buffer": [vp, ctypes.POINTER(vp), ctypes.POINTER(i64)],
        "b200_flat_buffer": [vp, ctypes.c_int, ctypes.POINTER(vp), ctypes.POINTER(i64)],
        "b200_loss": [vp, ctypes.POINTER(f32)],
        "b200_loss_of": [vp, ctypes.c_int, ctypes.POINTER(f32)],
        "b200_forward": [vp, ctypes.c_int, vp],
        "b200_sync": [vp],
        "b200_checkpoint_save": [vp, cp],
        "b200_checkpoint_load": [vp, cp],
        "b200_net_tensor_shape": [vp, cp, ctypes.POINTER(i64), ctypes.POINTER(i64)],
        "b200_quantise": [vp, i64, i32, i32, i32, vp],
        "b200_transpose": [vp, i64, i64, vp],
        "b200_saved_format_size": [vp, ctypes.POINTER(CSavedFormat), i32, i32, ctypes.POINTER(i64)],
        "b200_saved_format_write": [vp, ctypes.POINTER(CSavedFormat), i32, i32, vp, i64],
        "b200_save_quantised": [vp, ctypes.POINTER(CSavedFormat), i32, cp],
        "b200_save_unquantised": [vp, ctypes.POINTER(CSavedFormat), i32, cp],
        "b200_get_timings": [vp, ctypes.POINTER(CTimings)],
        "b200_net_get_activation": [vp, ctypes.c_int, vp, i64],
        "b200_net_get_stat": [vp, cp, ctypes.POINTER(i64)],
        "b200_op_ft_forward": [ctypes.c_int, vp, ctypes.POINTER(CFtOp)],
        "b200_op_ft_forward_noalloc": [ctypes.c_int, vp, ctypes.POINTER(CFtOp)],
        "b200_map_chess768": [vp, i32, vp, vp, i32],
        "b200_map_chess_buckets_mirrored": [vp, i32, vp, vp, vp, i32],
        "b200_map_ataxx147": [vp, i32, vp, vp, i32],
        "b200_material_count": [vp, i32, i32, vp],
        "b200_make_targets": [vp, i32, f32, f32, vp],
        "b200_set_host_threads": [i32],
        "b200_probe_bandwidth": [ctypes.c_int, ctypes.c_int, i64, ctypes.c_int, ctypes.POINTER(ctypes.c_double)],
        "b200_pack_indices_u16": [vp, i64, vp],
        "b200_unpack_indices_u16": [vp, i64, vp],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = ctypes.c_int
    lib.b200_quant_size.argtypes = [i32]
    lib.b200_quant_size.restype = i64
    _lib = lib
    return lib


def check(rc: int) -> int:
    if rc < 0:
        raise B200Error(rc, load().b200_last_error().decode())
    return rc
