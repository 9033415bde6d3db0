"""ctypes view of ``include/onyxia_cuda.h``.

The shared libraries are built in-tree by ``onyxia_b200.build``; loading fails
loudly when they are missing — there is no Python or CPU fallback for the
device path.
"""
from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT_DIR = os.path.dirname(PKG_DIR)

OX_MAX_TERM_SYMS = 6


class DimTerm(C.Structure):
    _fields_ = [("coeff", C.c_int64), ("n_syms", C.c_int32), ("syms", C.c_int32 * OX_MAX_TERM_SYMS)]


class DimExprC(C.Structure):
    _fields_ = [("terms", C.POINTER(DimTerm)), ("n_terms", C.c_int32)]


class SliceSpecC(C.Structure):
    _fields_ = [("axis", C.c_uint64), ("start", DimExprC), ("end", DimExprC), ("step", C.c_int64)]


class PrimDesc(C.Structure):
    _fields_ = [
        ("kind", C.c_int32), ("op", C.c_int32), ("dtype", C.c_int32),
        ("trans_a", C.c_int32), ("trans_b", C.c_int32), ("keepdims", C.c_int32),
        ("axes", C.POINTER(C.c_uint64)), ("n_axes", C.c_int32),
        ("shape", C.POINTER(DimExprC)), ("n_shape", C.c_int32),
        ("axis", C.c_uint64),
        ("specs", C.POINTER(SliceSpecC)), ("n_specs", C.c_int32),
        ("len", DimExprC), ("block_size", C.c_uint64),
    ]


class AttrC(C.Structure):
    _fields_ = [
        ("name", C.c_char_p), ("kind", C.c_int32), ("i", C.c_int64), ("f", C.c_double),
        ("s", C.c_char_p), ("ints", C.POINTER(C.c_int64)), ("floats", C.POINTER(C.c_double)),
        ("n", C.c_int32),
    ]


class TensorTypeC(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("dims", C.POINTER(DimExprC)), ("rank", C.c_int32)]


class BackendOptions(C.Structure):
    _fields_ = [
        ("without_fused_kernels", C.c_int32), ("disable_graphs", C.c_int32),
        ("disable_pattern_fusion", C.c_int32), ("disable_persistent_step", C.c_int32), ("reserved", C.c_int32 * 4),
    ]


class KernelTiming(C.Structure):
    _fields_ = [("kernel", C.c_char_p), ("node", C.c_char_p), ("time_ns", C.c_uint64)]


_P = C.c_void_p
_i32p = C.POINTER(C.c_int32)
_u64p = C.POINTER(C.c_uint64)

# name -> (restype, argtypes); every symbol declared in include/onyxia_cuda.h.
SIGNATURES = {
    "ox_last_error": (C.c_char_p, []),
    "ox_module_new": (_P, []),
    "ox_module_free": (None, [_P]),
    "ox_module_clone": (_P, [_P]),
    "ox_module_tp_partition": (C.c_int32, [_P, C.c_int32, C.c_int32, C.POINTER(_P)]),
    "ox_module_tp_stats": (None, [_P, C.c_int32, C.POINTER(C.c_uint64)]),
    "ox_module_intern_symbol": (C.c_int32, [_P, C.c_char_p]),
    "ox_module_add_const": (C.c_int32, [_P, C.c_int32, _u64p, C.c_int32, _P, C.c_size_t, C.c_int32, _i32p]),
    "ox_module_add_input": (C.c_int32, [_P, C.c_char_p, C.c_int32, C.POINTER(DimExprC), C.c_int32, _i32p]),
    "ox_module_add_prim": (C.c_int32, [_P, C.POINTER(PrimDesc), _i32p, C.c_int32, _i32p]),
    "ox_module_add_composite": (C.c_int32, [_P, C.c_char_p, C.POINTER(AttrC), C.c_int32, _i32p, C.c_int32,
                                            C.POINTER(TensorTypeC), C.c_int32, _i32p]),
    "ox_module_add_output": (C.c_int32, [_P, C.c_char_p, C.c_int32]),
    "ox_module_add_constraint": (C.c_int32, [_P, C.POINTER(DimExprC), C.POINTER(DimExprC), C.c_char_p]),
    "ox_module_set_loc": (None, [_P, C.c_char_p, C.c_char_p]),
    "ox_module_validate": (C.c_int32, [_P]),
    "ox_module_inline_composites": (C.c_int32, [_P, C.POINTER(C.c_char_p), C.c_int32]),
    "ox_module_fold_transposes": (C.c_int32, [_P]),
    "ox_module_num_nodes": (C.c_int32, [_P]),
    "ox_module_num_values": (C.c_int32, [_P]),
    "ox_module_num_inputs": (C.c_int32, [_P]),
    "ox_module_num_outputs": (C.c_int32, [_P]),
    "ox_module_input_name": (C.c_char_p, [_P, C.c_int32]),
    "ox_module_output_name": (C.c_char_p, [_P, C.c_int32]),
    "ox_module_input_desc": (C.c_int32, [_P, C.c_int32, _i32p, _i32p]),
    "ox_module_eval_input_shape": (C.c_int32, [_P, C.c_int32, C.POINTER(C.c_char_p), _u64p, C.c_int32, _u64p]),
    "ox_module_node_op": (C.c_char_p, [_P, C.c_int32]),
    "ox_module_value_type_str": (C.c_char_p, [_P, C.c_int32]),
    "ox_backend_create": (C.c_int32, [_i32p, C.c_int32, C.POINTER(_P)]),
    "ox_backend_create_ex": (C.c_int32, [_i32p, C.c_int32, C.POINTER(BackendOptions), C.POINTER(_P)]),
    "ox_backend_free": (None, [_P]),
    "ox_backend_supports": (C.c_int32, [_P, C.c_char_p]),
    "ox_backend_prepare": (C.c_int32, [_P, _P, C.POINTER(_P)]),
    "ox_session_free": (None, [_P]),
    "ox_session_upload": (C.c_int32, [_P, C.c_int32, _u64p, C.c_int32, _P, C.c_size_t, C.POINTER(_P)]),
    "ox_session_run": (C.c_int32, [_P, C.POINTER(C.c_char_p), C.POINTER(_P), C.c_int32, C.POINTER(C.c_char_p),
                                   C.POINTER(_P), C.c_int32, _i32p]),
    "ox_session_num_outputs": (C.c_int32, [_P]),
    "ox_session_download": (C.c_int32, [_P, _P, _P, C.c_size_t, C.POINTER(C.c_size_t)]),
    "ox_tensor_clone": (_P, [_P]),
    "ox_tensor_release": (None, [_P]),
    "ox_tensor_describe": (C.c_int32, [_P, _i32p, _u64p, C.c_int32, _i32p]),
    "ox_tensor_nbytes": (C.c_size_t, [_P]),
    "ox_session_wait_idle": (C.c_int32, [_P]),
    "ox_session_resident_bytes": (C.c_uint64, [_P]),
    "ox_session_peak_resident_bytes": (C.c_uint64, [_P]),
    "ox_session_pool_stats": (None, [_P, _u64p, _u64p]),
    "ox_session_enable_profiling": (C.c_int32, [_P, C.c_int32]),
    "ox_session_take_timings": (C.c_int32, [_P, C.POINTER(KernelTiming), C.c_int32]),
    "ox_session_timer_start": (C.c_int32, [_P]),
    "ox_session_timer_stop": (C.c_int32, [_P, C.POINTER(C.c_float)]),
    "ox_session_launch_count": (C.c_uint64, [_P]),
    "ox_session_plan_stats": (None, [_P, _u64p]),
    "ox_session_argmax_last": (C.c_int32, [_P, _P, C.POINTER(_P)]),
    "ox_session_argmax_last_into": (C.c_int32, [_P, _P, _P]),
    "ox_session_sample_last": (C.c_int32, [_P, _P, C.c_float, C.c_int64, C.c_float, C.POINTER(C.c_float), C.c_size_t, C.POINTER(_P)]),
    "ox_llm_create": (C.c_int32, [_P, C.c_int64, C.POINTER(_P)]),
    "ox_llm_free": (None, [_P]),
    "ox_llm_sequence_length": (C.c_int64, [_P]),
    "ox_llm_logits_dtype": (C.c_int32, [_P]),
    "ox_llm_reset": (None, [_P]),
    "ox_llm_step": (C.c_int32, [_P, C.POINTER(C.c_int64), C.c_int32, C.POINTER(C.c_int64), C.c_void_p, C.c_size_t,
                                C.POINTER(C.c_size_t)]),
    "ox_llm_generate": (C.c_int32, [_P, C.POINTER(C.c_int64), C.c_int32, C.c_int32, C.POINTER(C.c_int64)]),
    "ox_llm_step_sampled": (C.c_int32, [_P, C.POINTER(C.c_int64), C.c_int32, C.c_float, C.c_int64, C.c_float, C.c_float,
                                        C.POINTER(C.c_int64)]),
    "ox_tp_unique_id": (C.c_int32, [C.c_char_p, C.POINTER(C.c_uint8)]),
    "ox_backend_peer_allreduce": (C.c_int32, [_P]),
    "ox_backend_join_tp": (C.c_int32, [_P, C.c_int32, C.c_int32, C.POINTER(C.c_uint8), C.c_char_p]),
}

# Symbols implemented by the host-only IR library (the rest need the CUDA one).
IR_SYMBOLS = [n for n in SIGNATURES if n.startswith("ox_module_")] + ["ox_last_error"]


def _bind(lib, names):
    for name in names:
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype, fn.argtypes = SIGNATURES[name]
    return lib


_ir = None
_cuda = None


def ir_path() -> str:
    return os.path.join(PKG_DIR, "libonyxia_ir.so")


def cuda_path() -> str:
    return os.path.join(PKG_DIR, "libonyxia_cuda.so")


def ir_lib():
    """The host-only IR library (module construction, validation, legalisation)."""
    global _ir
    if _ir is None:
        if not os.path.exists(ir_path()):
            raise ImportError(f"{ir_path()} is missing: build it with `python -m onyxia_b200.build`")
        _ir = _bind(C.CDLL(ir_path(), mode=C.RTLD_GLOBAL), IR_SYMBOLS)
    return _ir


def cuda_lib():
    """The CUDA backend library. No fallback: a missing library is an error."""
    global _cuda
    if _cuda is None:
        ir_lib()
        if not os.path.exists(cuda_path()):
            raise ImportError(f"{cuda_path()} is missing: build it with `python -m onyxia_b200.build` "
                              "(the device path has no CPU fallback)")
        _cuda = _bind(C.CDLL(cuda_path(), mode=C.RTLD_GLOBAL), list(SIGNATURES))
    return _cuda


class OnyxiaError(RuntimeError):
    """An ``onyxia_ir::Error`` carried across the C boundary."""

    KINDS = {1: "Shape", 2: "InvalidGraph", 3: "DType", 4: "Attribute", 5: "Binding", 6: "Interp",
             7: "Unsupported", 8: "Runtime"}

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status
        self.kind = self.KINDS.get(status, "Unknown")


def check(status: int) -> None:
    if status != 0:
        msg = ir_lib().ox_last_error()
        raise OnyxiaError(status, msg.decode("utf-8", "replace") if msg else "unknown error")
