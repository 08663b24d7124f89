"""ctypes binding of ``libaarambh_b200.so`` (the C ABI in ``include/aarambh_b200.h``).

The library is the only compute path: importing this module without the built
shared object raises, and nothing here falls back to PyTorch or the CPU.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libaarambh_b200.so")

OK = 0
F32, F16, BF16 = 0, 1, 2
KV_F32, KV_BF16, KV_INT8 = 0, 1, 2
FMT_I8, FMT_I4_AFFINE, FMT_Q4KM, FMT_W4A16 = 0, 1, 2, 3

STATUS_NAMES = {
    0: "OK", -1: "BAD_SHAPE", -2: "BAD_ALIGN", -3: "BAD_DTYPE", -4: "CAPACITY", -5: "CUDA_ERROR",
    -6: "TIMEOUT", -7: "BAD_ARG", -8: "UNSUPPORTED",
}


class Ab2Error(RuntimeError):
    """A failed library call; ``status`` is the ab2_status code."""

    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python aarambh-ai_b200/build.py` "
        "(there is no fallback path)")

lib = C.CDLL(LIB_PATH)

_p = C.c_void_p
_i = C.c_int
_f = C.c_float
_pp = C.POINTER(C.c_void_p)

# name -> (argtypes, restype); every symbol declared in include/aarambh_b200.h.
SIGNATURES = {
    "ab2_version": ([], _i),
    "ab2_last_error": ([], C.c_char_p),
    "ab2_device_status": ([C.POINTER(_i)], _i),
    "ab2_qweight_from_i8_tensor": ([_pp, _p, _f, _i, _i], _i),
    "ab2_qweight_from_i8_channel": ([_pp, _p, _p, _i, _i], _i),
    "ab2_qweight_from_i4_affine": ([_pp, _p, _p, _p, _i, _i, _i], _i),
    "ab2_qweight_from_q4km_blocks": ([_pp, _p, _i, _i], _i),
    "ab2_qweight_from_w4a16_gptq": ([_pp, _p, _p, _p, _i, _i, _i], _i),
    "ab2_qweight_from_w4a16_awq": ([_pp, _p, _p, _p, _i, _i, _i], _i),
    "ab2_qweight_quantise_i8": ([_pp, _p, _i, _i, _i, _p], _i),
    "ab2_qweight_quantise_i4_affine": ([_pp, _p, _i, _i, _i, _p], _i),
    "ab2_qweight_quantise_q4km": ([_pp, _p, _i, _i, _p], _i),
    "ab2_qweight_quantise_w4a16": ([_pp, _p, _i, _i, _i, _p], _i),
    "ab2_qweight_concat_rows": ([_pp, _pp, _i], _i),
    "ab2_qweight_interleave_gate_up": ([_pp, _p, _p], _i),
    "ab2_qweight_destroy": ([_p], _i),
    "ab2_qweight_shape": ([_p, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)], _i),
    "ab2_qweight_nbytes": ([_p, C.POINTER(C.c_size_t)], _i),
    "ab2_qweight_export": ([_p, _p, _p, _p], _i),
    "ab2_qweight_dequant": ([_p, _p, _i, _p], _i),
    "ab2_qlinear_forward": ([_p, _p, _i, _i, _p, _p], _i),
    "ab2_rms_norm": ([_p, _p, _p, _i, _i, _f, _i, _p], _i),
    "ab2_rope_apply": ([_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p], _i),
    "ab2_swiglu": ([_p, _p, _p, C.c_size_t, _i, _p], _i),
    "ab2_argmax": ([_p, _i, _i, _i, _p, _p], _i),
    "ab2_embedding_forward": ([_p, _p, _i, _p, _i, _p], _i),
    "ab2_kv_create": ([_pp, _i, _i, _i, _i, _i, _i, _i], _i),
    "ab2_kv_destroy": ([_p], _i),
    "ab2_kv_update": ([_p, _p, _p, _i, _i, _i, _i, _p], _i),
    "ab2_kv_append": ([_p, _i, _p, _p, _i, _i, _i, _i, _p, _p, _p, _i, _p], _i),
    "ab2_kv_commit": ([_p, _i, _i, _i, _p], _i),
    "ab2_kv_truncate": ([_p, _i, _i, _p], _i),
    "ab2_kv_clear": ([_p, _p], _i),
    "ab2_kv_seq_len": ([_p, _i, C.POINTER(_i)], _i),
    "ab2_kv_capacity": ([_p, C.POINTER(_i)], _i),
    "ab2_kv_clone": ([_pp, _p, _p], _i),
    "ab2_kv_read": ([_p, _i, _i, _p, _p, _p], _i),
    "ab2_attention_decode": ([_p, _i, _p, _p, _i, _i, _f, _i, _p], _i),
    "ab2_attention_decode_static": ([_p, _i, _p, _p, _i, _i, _f, _i, _p], _i),
    "ab2_attention_cached": ([_p, _i, _p, _p, _i, _i, _i, _f, _i, _p], _i),
    "ab2_attention_causal": ([_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _i, _p], _i),
    "ab2_model_create": ([_pp, _p, _i, _i], _i),
    "ab2_model_destroy": ([_p], _i),
    "ab2_model_set_linear": ([_p, _i, _i, _p], _i),
    "ab2_model_set_norm": ([_p, _i, _i, _p], _i),
    "ab2_model_finalize": ([_p], _i),
    "ab2_model_set_tp": ([_p, _p], _i),
    "ab2_tp_unique_id": ([_p], _i),
    "ab2_tp_create": ([_pp, _i, _i, _p], _i),
    "ab2_tp_destroy": ([_p], _i),
    "ab2_tp_all_reduce": ([_p, _p, C.c_size_t, _i, _p], _i),
    "ab2_tp_peer_export": ([_p, C.c_size_t, _p], _i),
    "ab2_tp_peer_attach": ([_p, _p], _i),
    "ab2_tp_peer_block": ([_p, _pp, _p], _i),
    "ab2_tp_peer_attach_ptrs": ([_p, _p], _i),
    "ab2_tp_set_wait_limit_ns": ([_p, C.c_ulonglong], _i),
    "ab2_tp_peer_reset": ([_p], _i),
    "ab2_tp_peer_deposit": ([_p, _p, C.c_size_t, _p], _i),
    "ab2_tp_peer_reduce_add": ([_p, _p, C.c_size_t, _p], _i),
    "ab2_model_rope_tables": ([_p, _pp, _pp], _i),
    "ab2_model_forward": ([_p, _p, _p, _i, _i, _i, _p, _i, _p, _p, _p], _i),
    "ab2_model_decode_step": ([_p, _p, _p, _i, _i, _p, _p, _p], _i),
    "ab2_model_decode_step_host": ([_p, _p, _p, _i, _i, _p, _p], _i),
    "ab2_model_step_trace": ([_p, _p, _i, _p], _i),
    "ab2_model_forward_rows": ([_p, _p, _p, _i, _p, _i, _i, _p, _p, _p], _i),
    "ab2_model_decode_step_rows": ([_p, _p, _p, _p, _i, _p, _p, _p], _i),
}


class ModelConfig(C.Structure):
    """ab2_model_config."""
    _fields_ = [("n_layers", _i), ("d_model", _i), ("n_heads", _i), ("n_kv_heads", _i),
                ("head_dim", _i), ("ffn_hidden", _i), ("vocab", _i), ("max_seq", _i),
                ("rms_eps", _f), ("rope_theta", C.c_double), ("tied", _i)]


def _declare():
    for name, (argtypes, restype) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype


_declare()


def check(status: int) -> None:
    if status != OK:
        raise Ab2Error(status, lib.ab2_last_error().decode("utf-8", "replace"))


def device_status() -> int:
    """Synchronises and returns the device status word (0, or a negative ab2_status)."""
    out = C.c_int(0)
    check(lib.ab2_device_status(C.byref(out)))
    return out.value
