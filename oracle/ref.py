"""TEST INFRASTRUCTURE — Python access to the CPU oracle (``libonyxia_ref.so``).

Mirrors ``onyxia_backend_ref`` (crates/onyxia-backend-ref/src/lib.rs:21-107):
``RefBackend.prepare`` inlines every composite, ``RefSession.run`` interprets.
Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this module; the device path never does.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from onyxia_b200 import _ffi
from onyxia_b200.ir import HostTensor, Module

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None


def lib():
    global _lib
    if _lib is None:
        _ffi.ir_lib()
        path = os.path.join(_HERE, "libonyxia_ref.so")
        if not os.path.exists(path):
            raise ImportError(f"{path} is missing: run `make -C oracle` (or `python -m onyxia_b200.build`)")
        l = C.CDLL(path, mode=C.RTLD_GLOBAL)
        P = C.c_void_p
        l.oxref_set_threads.argtypes = [C.c_int]
        l.oxref_get_threads.restype = C.c_int
        l.oxref_prepare.argtypes = [P, C.POINTER(P)]
        l.oxref_session_free.argtypes = [P]
        l.oxref_session_num_nodes.argtypes = [P]
        l.oxref_run.argtypes = [P, C.POINTER(C.c_char_p), C.POINTER(C.c_int32), C.POINTER(C.POINTER(C.c_uint64)),
                                C.POINTER(C.c_int32), C.POINTER(P), C.POINTER(C.c_size_t), C.c_int32, C.POINTER(P)]
        for name, res in [("oxref_result_count", C.c_int), ("oxref_result_name", C.c_char_p),
                          ("oxref_result_dtype", C.c_int), ("oxref_result_rank", C.c_int),
                          ("oxref_result_data", P), ("oxref_result_nbytes", C.c_size_t)]:
            getattr(l, name).restype = res
        l.oxref_result_count.argtypes = [P]
        for name in ("oxref_result_name", "oxref_result_dtype", "oxref_result_rank", "oxref_result_data",
                     "oxref_result_nbytes"):
            getattr(l, name).argtypes = [P, C.c_int]
        l.oxref_result_shape.argtypes = [P, C.c_int, C.POINTER(C.c_uint64)]
        l.oxref_result_free.argtypes = [P]
        l.oxref_f64_to_f16.argtypes = [C.c_double]
        l.oxref_f64_to_f16.restype = C.c_uint16
        l.oxref_f16_to_f64.argtypes = [C.c_uint16]
        l.oxref_f16_to_f64.restype = C.c_double
        _lib = l
    return _lib


ALLREDUCE_HOOK = C.CFUNCTYPE(None, C.c_void_p, C.c_uint64, C.c_int32)
_hook_keepalive = None


def set_allreduce_hook(fn) -> None:
    """Install the function the interpreter calls at every ``onyxia.AllReduce`` node:
    ``fn(numpy_view)`` must replace the view's content by its sum over the tensor-parallel
    ranks (the test that runs the ranks — as threads or as processes — supplies it).
    ``None`` removes the hook."""
    global _hook_keepalive
    if fn is None:
        lib().oxref_set_allreduce_hook.argtypes = [C.c_void_p]
        lib().oxref_set_allreduce_hook(None)
        _hook_keepalive = None
        return
    import numpy as np
    from onyxia_b200 import ir
    np_of = {ir.F32: np.float32, ir.F16: np.float16, ir.I64: np.int64, ir.I32: np.int32}

    def thunk(data, count, dtype):
        arr = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint8)), shape=(count * np.dtype(np_of[dtype]).itemsize,))
        fn(arr.view(np_of[dtype]))

    cb = ALLREDUCE_HOOK(thunk)
    lib().oxref_set_allreduce_hook.argtypes = [ALLREDUCE_HOOK]
    lib().oxref_set_allreduce_hook(cb)
    _hook_keepalive = cb


def set_threads(n: int) -> None:
    """1 = the reference's single-threaded behaviour; more threads split big
    loops over outputs without changing any accumulation order."""
    lib().oxref_set_threads(int(n))


class RefSession:
    def __init__(self, handle):
        self._h = handle

    @property
    def num_nodes(self) -> int:
        return lib().oxref_session_num_nodes(self._h)

    def upload(self, t: HostTensor) -> HostTensor:
        return t

    def download(self, t: HostTensor) -> HostTensor:
        return t

    def run(self, inputs) -> list:
        """inputs: dict or list of (name, HostTensor); returns [(name, HostTensor)] in signature order."""
        items = list(inputs.items()) if isinstance(inputs, dict) else list(inputs)
        n = len(items)
        names = (C.c_char_p * max(n, 1))(*[k.encode() for k, _ in items])
        dtypes = (C.c_int32 * max(n, 1))(*[t.dtype for _, t in items])
        ranks = (C.c_int32 * max(n, 1))(*[len(t.shape) for _, t in items])
        shape_arrs = [(C.c_uint64 * max(len(t.shape), 1))(*t.shape) for _, t in items]
        shapes = (C.POINTER(C.c_uint64) * max(n, 1))(*[C.cast(a, C.POINTER(C.c_uint64)) for a in shape_arrs])
        datas = (C.c_void_p * max(n, 1))(*[t.data.ctypes.data for _, t in items])
        nbytes = (C.c_size_t * max(n, 1))(*[t.data.size for _, t in items])
        res = C.c_void_p()
        _ffi.check(lib().oxref_run(self._h, names, dtypes, shapes, ranks, datas, nbytes, n, C.byref(res)))
        out = []
        l = lib()
        try:
            for i in range(l.oxref_result_count(res)):
                rank = l.oxref_result_rank(res, i)
                shp = (C.c_uint64 * max(rank, 1))()
                l.oxref_result_shape(res, i, shp)
                nb = l.oxref_result_nbytes(res, i)
                buf = np.empty(nb, dtype=np.uint8)
                if nb:
                    C.memmove(buf.ctypes.data, l.oxref_result_data(res, i), nb)
                out.append((l.oxref_result_name(res, i).decode(),
                            HostTensor(l.oxref_result_dtype(res, i), [shp[d] for d in range(rank)], buf)))
        finally:
            l.oxref_result_free(res)
        return out

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                lib().oxref_session_free(self._h)
            except Exception:
                pass
            self._h = None


class RefBackend:
    """≙ ``RefBackend``: no fused kernels, everything runs through decompositions."""

    def supports(self, composite: str) -> bool:
        return False

    def prepare(self, module: Module) -> RefSession:
        h = C.c_void_p()
        _ffi.check(lib().oxref_prepare(module._take(), C.byref(h)))
        return RefSession(h)


def run_once(module: Module, inputs) -> list:
    """≙ ``onyxia_backend_ref::run_once`` (lib.rs:96-107)."""
    return RefBackend().prepare(module).run(inputs)
