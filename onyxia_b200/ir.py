"""Python mirror of the reference's module-construction API.

Names follow ``onyxia_ir``: :class:`GraphBuilder` (crates/onyxia-ir/src/builder.rs),
:class:`DimExpr` (dim.rs), :class:`HostTensor` ≙ ``interp::Tensor``
(interp.rs:29-49). Every call goes through the C ABI of
``include/onyxia_cuda.h``; nothing is evaluated in Python.
"""
from __future__ import annotations

import ctypes as C
from typing import Iterable, Sequence

import numpy as np

from . import _ffi
from ._ffi import check

# ── dtypes (crates/onyxia-ir/src/types.rs:13-26) ─────────────────────────
F32, F16, I64, I32, U32, U8, I8, BOOL, U4, I4 = range(10)
DTYPE_NAMES = ["f32", "f16", "i64", "i32", "u32", "u8", "i8", "bool", "u4", "i4"]
DTYPE_BITS = [32, 16, 64, 32, 32, 8, 8, 8, 4, 4]
_NP = {F32: np.float32, F16: np.float16, I64: np.int64, I32: np.int32, U32: np.uint32, U8: np.uint8,
       I8: np.int8, BOOL: np.bool_}
_FROM_NP = {np.dtype(v): k for k, v in _NP.items()}


def storage_bytes(dtype: int, numel: int) -> int:
    return (numel * DTYPE_BITS[dtype] + 7) // 8


# ── operator codes (crates/onyxia-ir/src/prim.rs:27-107) ─────────────────
NEG, ABS, SQRT, RSQRT, EXP, LOG, SIN, COS, TANH, ERF, FLOOR, CEIL, NOT = range(13)
ADD, SUB, MUL, DIV, POW, MAX, MIN, AND, OR, XOR = range(10)
EQ, NE, LT, LE, GT, GE = range(6)
SUM, MEAN, RMAX, RMIN, PROD = range(5)
(P_UNARY, P_BINARY, P_COMPARE, P_SELECT, P_CAST, P_MATMUL, P_REDUCE, P_RESHAPE, P_TRANSPOSE, P_BROADCAST,
 P_CONCAT, P_SLICE, P_GATHER, P_SCATTER, P_IOTA, P_DIM_VALUES, P_DEQUANTIZE) = range(17)


class DimExpr:
    """Integer polynomial over dimension symbols (crates/onyxia-ir/src/dim.rs:143-308)."""

    __slots__ = ("terms",)

    def __init__(self, terms=None):
        # {sorted tuple of symbol ids: coeff}
        self.terms = {k: v for k, v in (terms or {}).items() if v != 0}

    @staticmethod
    def of(x) -> "DimExpr":
        if isinstance(x, DimExpr):
            return x
        return DimExpr({(): int(x)})

    @staticmethod
    def sym(sym_id: int) -> "DimExpr":
        return DimExpr({(int(sym_id),): 1})

    def __add__(self, o):
        o = DimExpr.of(o)
        t = dict(self.terms)
        for k, v in o.terms.items():
            t[k] = t.get(k, 0) + v
        return DimExpr(t)

    __radd__ = __add__

    def __sub__(self, o):
        o = DimExpr.of(o)
        t = dict(self.terms)
        for k, v in o.terms.items():
            t[k] = t.get(k, 0) - v
        return DimExpr(t)

    def __rsub__(self, o):
        return DimExpr.of(o) - self

    def __mul__(self, o):
        o = DimExpr.of(o)
        t = {}
        for ka, va in self.terms.items():
            for kb, vb in o.terms.items():
                k = tuple(sorted(ka + kb))
                t[k] = t.get(k, 0) + va * vb
        return DimExpr(t)

    __rmul__ = __mul__

    def __eq__(self, o):
        return isinstance(o, (DimExpr, int)) and self.terms == DimExpr.of(o).terms

    def __hash__(self):
        return hash(tuple(sorted(self.terms.items())))

    def div_exact(self, divisor) -> "DimExpr | None":
        """Exact division by a monomial (dim.rs:254-280): None when the divisor is not a single term or some term's
        coefficient or symbols are not divisible by it."""
        d = DimExpr.of(divisor)
        if len(d.terms) != 1:
            return None
        (dsyms, dcoeff), = d.terms.items()
        out = {}
        for syms, coeff in self.terms.items():
            if coeff % dcoeff:
                return None
            rest = list(syms)
            for sy in dsyms:
                if sy not in rest:
                    return None
                rest.remove(sy)
            out[tuple(rest)] = out.get(tuple(rest), 0) + coeff // dcoeff
        return DimExpr(out)

    def as_const(self):
        if not self.terms:
            return 0
        if list(self.terms) == [()] and self.terms[()] >= 0:
            return self.terms[()]
        return None

    def to_c(self, keep: list) -> _ffi.DimExprC:
        n = len(self.terms)
        arr = (_ffi.DimTerm * max(n, 1))()
        for i, (syms, coeff) in enumerate(self.terms.items()):
            if len(syms) > _ffi.OX_MAX_TERM_SYMS:
                raise ValueError("dim term has too many symbols")
            arr[i].coeff = coeff
            arr[i].n_syms = len(syms)
            for j, s in enumerate(syms):
                arr[i].syms[j] = s
        keep.append(arr)
        return _ffi.DimExprC(C.cast(arr, C.POINTER(_ffi.DimTerm)), n)

    def __repr__(self):
        return "DimExpr(%r)" % (self.terms,)


def _shape_to_c(shape: Sequence, keep: list):
    n = len(shape)
    arr = (_ffi.DimExprC * max(n, 1))()
    for i, d in enumerate(shape):
        arr[i] = DimExpr.of(d).to_c(keep)
    keep.append(arr)
    return C.cast(arr, C.POINTER(_ffi.DimExprC)), n


class HostTensor:
    """dtype + shape + little-endian storage bytes ≙ ``interp::Tensor``."""

    def __init__(self, dtype: int, shape: Sequence[int], data):
        self.dtype = int(dtype)
        self.shape = tuple(int(d) for d in shape)
        buf = np.ascontiguousarray(np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data)
        if buf.dtype != np.uint8:
            buf = buf.view(np.uint8)
        self.data = buf.reshape(-1)
        expect = storage_bytes(self.dtype, int(np.prod(self.shape, dtype=np.int64)))
        if self.data.size != expect:
            raise ValueError(f"tensor data size mismatch: {self.data.size} bytes for "
                             f"{DTYPE_NAMES[self.dtype]}{list(self.shape)} (expected {expect})")

    @staticmethod
    def from_numpy(a: np.ndarray) -> "HostTensor":
        a = np.ascontiguousarray(a)
        if a.dtype not in _FROM_NP:
            raise TypeError(f"unsupported numpy dtype {a.dtype}")
        return HostTensor(_FROM_NP[a.dtype], a.shape, a.view(np.uint8).reshape(-1))

    @staticmethod
    def packed_u4(values: np.ndarray, shape: Sequence[int], dtype: int = U4) -> "HostTensor":
        """Pack integer values (0..15 or -8..7) two per byte, low nibble first."""
        v = np.asarray(values).astype(np.int64).reshape(-1) & 0xF
        if v.size % 2:
            v = np.concatenate([v, [0]])
        packed = (v[0::2] | (v[1::2] << 4)).astype(np.uint8)
        return HostTensor(dtype, shape, packed)

    @property
    def numel(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64))

    def numpy(self) -> np.ndarray:
        """Logical values; packed nibbles are unpacked to int8/uint8."""
        if self.dtype in (U4, I4):
            lo, hi = self.data & 0xF, self.data >> 4
            v = np.stack([lo, hi], axis=1).reshape(-1)[: self.numel]
            if self.dtype == I4:
                v = ((v.astype(np.int8) << 4) >> 4)
            return v.reshape(self.shape)
        return self.data.view(_NP[self.dtype]).reshape(self.shape)

    def __repr__(self):
        return f"HostTensor({DTYPE_NAMES[self.dtype]}{list(self.shape)})"


class Module:
    """An owned ``ox_module*``. ``prepare`` calls consume it."""

    def __init__(self, handle, keep=None):
        self._h = handle
        self._keep = keep or []  # borrowed constant buffers

    def _take(self):
        if self._h is None:
            raise RuntimeError("module was already consumed by prepare()")
        h, self._h = self._h, None
        return h

    @property
    def handle(self):
        if self._h is None:
            raise RuntimeError("module was already consumed by prepare()")
        return self._h

    def clone(self) -> "Module":
        return Module(_ffi.ir_lib().ox_module_clone(self.handle), self._keep)

    def tp_partition(self, tp: int, rank: int) -> "Module":
        """The module rank `rank` of `tp` tensor-parallel ranks executes (this module is left untouched)."""
        out = C.c_void_p()
        check(_ffi.ir_lib().ox_module_tp_partition(self.handle, tp, rank, C.byref(out)))
        return Module(out, self._keep)

    def tp_stats(self, tp: int) -> tuple:
        """(MatMulNBits nodes split along N, split along K, attention nodes split) for `tp` ranks."""
        out = (C.c_uint64 * 3)()
        _ffi.ir_lib().ox_module_tp_stats(self.handle, tp, out)
        return out[0], out[1], out[2]

    def validate(self) -> None:
        check(_ffi.ir_lib().ox_module_validate(self.handle))

    def inline_composites(self, keep: Iterable[str] = ()) -> "Module":
        names = [k.encode() for k in keep]
        arr = (C.c_char_p * max(len(names), 1))(*names)
        check(_ffi.ir_lib().ox_module_inline_composites(self.handle, arr, len(names)))
        return self

    def fold_transposes(self) -> bool:
        """Transposes of the last two axes that feed a MatMul become its trans flags (fold.rs:129-178)."""
        r = _ffi.ir_lib().ox_module_fold_transposes(self.handle)
        if r < 0:
            raise RuntimeError("fold_transposes failed")
        return r > 0

    @property
    def num_nodes(self) -> int:
        return _ffi.ir_lib().ox_module_num_nodes(self.handle)

    def node_ops(self) -> list:
        lib = _ffi.ir_lib()
        return [lib.ox_module_node_op(self.handle, i).decode() for i in range(self.num_nodes)]

    def input_names(self) -> list:
        lib = _ffi.ir_lib()
        return [lib.ox_module_input_name(self.handle, i).decode() for i in range(lib.ox_module_num_inputs(self.handle))]

    def output_names(self) -> list:
        lib = _ffi.ir_lib()
        return [lib.ox_module_output_name(self.handle, i).decode() for i in range(lib.ox_module_num_outputs(self.handle))]

    def input_desc(self, i: int):
        dt, rank = C.c_int32(), C.c_int32()
        check(_ffi.ir_lib().ox_module_input_desc(self.handle, i, C.byref(dt), C.byref(rank)))
        return dt.value, rank.value

    def eval_input_shape(self, i: int, bindings: dict) -> tuple:
        _, rank = self.input_desc(i)
        names = [k.encode() for k in bindings]
        arr = (C.c_char_p * max(len(names), 1))(*names)
        vals = (C.c_uint64 * max(len(names), 1))(*[int(v) for v in bindings.values()])
        out = (C.c_uint64 * max(rank, 1))()
        check(_ffi.ir_lib().ox_module_eval_input_shape(self.handle, i, arr, vals, len(names), out))
        return tuple(out[d] for d in range(rank))

    def value_type_str(self, v: int) -> str:
        s = _ffi.ir_lib().ox_module_value_type_str(self.handle, int(v))
        return s.decode() if s else "?"

    def __del__(self):
        if getattr(self, "_h", None) is not None:
            try:
                _ffi.ir_lib().ox_module_free(self._h)
            except Exception:
                pass
            self._h = None


class GraphBuilder:
    """Eagerly typed module construction ≙ ``onyxia_ir::GraphBuilder``."""

    def __init__(self):
        self._lib = _ffi.ir_lib()
        self._m = Module(self._lib.ox_module_new())

    # symbols / io
    def sym(self, name: str) -> DimExpr:
        return DimExpr.sym(self._lib.ox_module_intern_symbol(self._m.handle, name.encode()))

    def input(self, name: str, dtype: int, shape: Sequence) -> int:
        keep = []
        dims, rank = _shape_to_c(shape, keep)
        out = C.c_int32()
        check(self._lib.ox_module_add_input(self._m.handle, name.encode(), dtype, dims, rank, C.byref(out)))
        return out.value

    def output(self, name: str, value: int) -> None:
        check(self._lib.ox_module_add_output(self._m.handle, name.encode(), value))

    def constrain(self, left, right, context: str) -> None:
        keep = []
        l, r = DimExpr.of(left).to_c(keep), DimExpr.of(right).to_c(keep)
        check(self._lib.ox_module_add_constraint(self._m.handle, C.byref(l), C.byref(r), context.encode()))

    def set_loc(self, name: str | None, op_type: str | None = None) -> None:
        self._lib.ox_module_set_loc(self._m.handle, name.encode() if name else None,
                                    op_type.encode() if op_type else None)

    # constants
    def constant(self, t: HostTensor, borrow: bool = False) -> int:
        dims = (C.c_uint64 * max(len(t.shape), 1))(*t.shape)
        out = C.c_int32()
        ptr = t.data.ctypes.data_as(C.c_void_p)
        if borrow:
            self._m._keep.append(t.data)
        check(self._lib.ox_module_add_const(self._m.handle, t.dtype, dims, len(t.shape), ptr, t.data.size,
                                            1 if borrow else 0, C.byref(out)))
        return out.value

    def const_f32(self, values, dims) -> int:
        return self.constant(HostTensor.from_numpy(np.asarray(values, dtype=np.float32).reshape(dims)))

    def const_f16(self, values, dims) -> int:
        return self.constant(HostTensor.from_numpy(np.asarray(values, dtype=np.float16).reshape(dims)))

    def const_i64(self, values, dims) -> int:
        return self.constant(HostTensor.from_numpy(np.asarray(values, dtype=np.int64).reshape(dims)))

    # nodes
    def prim(self, kind: int, inputs: Sequence[int], *, op=0, dtype=F32, trans_a=False, trans_b=False,
             keepdims=False, axes=(), shape=(), axis=0, specs=(), length=0, block_size=0) -> int:
        keep = []
        d = _ffi.PrimDesc()
        d.kind, d.op, d.dtype = kind, op, dtype
        d.trans_a, d.trans_b, d.keepdims = int(trans_a), int(trans_b), int(keepdims)
        ax = (C.c_uint64 * max(len(axes), 1))(*[int(a) for a in axes])
        d.axes, d.n_axes = C.cast(ax, C.POINTER(C.c_uint64)), len(axes)
        d.shape, d.n_shape = _shape_to_c(shape, keep)
        d.axis = axis
        sp = (_ffi.SliceSpecC * max(len(specs), 1))()
        for i, (s_axis, start, end, step) in enumerate(specs):
            sp[i].axis = s_axis
            sp[i].start = DimExpr.of(start).to_c(keep)
            sp[i].end = DimExpr.of(end).to_c(keep)
            sp[i].step = step
        d.specs, d.n_specs = C.cast(sp, C.POINTER(_ffi.SliceSpecC)), len(specs)
        d.len = DimExpr.of(length).to_c(keep)
        d.block_size = block_size
        ins = (C.c_int32 * max(len(inputs), 1))(*inputs)
        out = C.c_int32()
        check(self._lib.ox_module_add_prim(self._m.handle, C.byref(d), ins, len(inputs), C.byref(out)))
        return out.value

    def composite(self, name: str, attrs: dict, inputs: Sequence[int], out_types: Sequence[tuple]) -> list:
        """``out_types`` = [(dtype, shape), …]; attrs values: int, float, str, bool, list."""
        keep = []
        n_attrs = len(attrs)
        arr = (_ffi.AttrC * max(n_attrs, 1))()
        for i, (k, v) in enumerate(attrs.items()):
            kb = k.encode()
            keep.append(kb)
            arr[i].name = kb
            if isinstance(v, bool):
                arr[i].kind, arr[i].i = 5, int(v)
            elif isinstance(v, int):
                arr[i].kind, arr[i].i = 0, v
            elif isinstance(v, float):
                arr[i].kind, arr[i].f = 2, v
            elif isinstance(v, str):
                sb = v.encode()
                keep.append(sb)
                arr[i].kind, arr[i].s = 4, sb
            elif isinstance(v, (list, tuple)) and all(isinstance(x, int) for x in v):
                a = (C.c_int64 * max(len(v), 1))(*v)
                keep.append(a)
                arr[i].kind, arr[i].ints, arr[i].n = 1, C.cast(a, C.POINTER(C.c_int64)), len(v)
            elif isinstance(v, (list, tuple)):
                a = (C.c_double * max(len(v), 1))(*[float(x) for x in v])
                keep.append(a)
                arr[i].kind, arr[i].floats, arr[i].n = 3, C.cast(a, C.POINTER(C.c_double)), len(v)
            else:
                raise TypeError(f"attribute {k!r}: unsupported value {v!r}")
        tys = (_ffi.TensorTypeC * max(len(out_types), 1))()
        for i, (dt, shape) in enumerate(out_types):
            tys[i].dtype = dt
            tys[i].dims, tys[i].rank = _shape_to_c(shape, keep)
        ins = (C.c_int32 * max(len(inputs), 1))(*inputs)
        outs = (C.c_int32 * max(len(out_types), 1))()
        check(self._lib.ox_module_add_composite(self._m.handle, name.encode(), arr, n_attrs, ins, len(inputs),
                                                tys, len(out_types), outs))
        return [outs[i] for i in range(len(out_types))]

    # sugar (crates/onyxia-ir/src/builder.rs:250-360)
    def unary(self, op, x): return self.prim(P_UNARY, [x], op=op)
    def binary(self, op, a, b): return self.prim(P_BINARY, [a, b], op=op)
    def add(self, a, b): return self.binary(ADD, a, b)
    def sub(self, a, b): return self.binary(SUB, a, b)
    def mul(self, a, b): return self.binary(MUL, a, b)
    def div(self, a, b): return self.binary(DIV, a, b)
    def cmp(self, op, a, b): return self.prim(P_COMPARE, [a, b], op=op)
    def select(self, c, a, b): return self.prim(P_SELECT, [c, a, b])
    def cast(self, x, to): return self.prim(P_CAST, [x], dtype=to)
    def matmul(self, a, b, trans_a=False, trans_b=False): return self.prim(P_MATMUL, [a, b], trans_a=trans_a, trans_b=trans_b)
    def reduce(self, op, x, axes, keepdims): return self.prim(P_REDUCE, [x], op=op, axes=axes, keepdims=keepdims)
    def reshape(self, x, shape): return self.prim(P_RESHAPE, [x], shape=shape)
    def transpose(self, x, perm): return self.prim(P_TRANSPOSE, [x], axes=perm)
    def broadcast(self, x, shape): return self.prim(P_BROADCAST, [x], shape=shape)
    def concat(self, xs, axis): return self.prim(P_CONCAT, list(xs), axis=axis)
    def slice(self, x, specs): return self.prim(P_SLICE, [x], specs=specs)
    def gather(self, data, indices, axis): return self.prim(P_GATHER, [data, indices], axis=axis)
    def scatter(self, data, indices, updates): return self.prim(P_SCATTER, [data, indices, updates])
    def iota(self, length, dtype): return self.prim(P_IOTA, [], length=length, dtype=dtype)
    def dim_values(self, exprs): return self.prim(P_DIM_VALUES, [], shape=exprs)
    def dequantize(self, data, scales, zp=None, *, block_size, out_shape):
        ins = [data, scales] + ([zp] if zp is not None else [])
        return self.prim(P_DEQUANTIZE, ins, block_size=block_size, shape=out_shape)

    def module(self) -> Module:
        return self._m

    def finish(self) -> Module:
        """Validate and hand over the module (builder.rs:245-248)."""
        self._m.validate()
        m, self._m = self._m, None
        return m
