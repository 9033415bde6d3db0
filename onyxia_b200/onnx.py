"""A minimal ONNX reader / writer and the lowering of the operators a quantised decoder export uses.

≙ ``crates/onyxia-onnx/src/parser.rs:17-117`` (ModelProto → graph) and the rules of
``crates/onyxia-lower/src/rules.rs:18-96``: one ``op_<Name>`` method per registered operator — the composites
(``Softmax``, ``Gelu``, ``Trilu``, ``SimplifiedLayerNormalization``, ``com.microsoft.MatMulNBits`` :890-940,
``com.microsoft.GroupQueryAttention`` :777-888, the two rotary embeddings) and the plain element-wise,
structural and reduction operators, plus ``Constant`` nodes (initializers spelled as nodes). There is no
``protoc`` and no ``onnx`` package here, so the protobuf wire format is read and written by hand
(varints, length-delimited fields); only the fields of ``onnx.proto`` that such graphs use are known.

Lowering conventions taken from the reference:

* shape arithmetic that an export spells with ``Shape → Gather → Cast`` is evaluated at lowering time
  into dimension expressions (the compile-time value domain, graph.rs:71-100) instead of nodes;
* ``MatMulNBits``: the packed ``uint8 [N, n_blocks, block/2]`` blob is reinterpreted as logical
  ``U4 [N, n_blocks, block]``, zero points as ``U4 [N, n_blocks]`` (needs an even block count per row);
* ``GroupQueryAttention``: inputs ``[q, k, v, past_k, past_v, seqlens_k][, cos, sin][, bias]``;
  ``total_sequence_length`` is not an operand — when it is a compile-time value it becomes the bind-time
  constraint *total = past + new*; ``present`` types are the past types with ``past + seq`` rows;
  softcap and explicit position ids with ``do_rotary`` are rejected.
"""
from __future__ import annotations

import struct

import numpy as np

from . import ir
from .ir import DimExpr, HostTensor

# onnx.proto TensorProto.DataType
_ONNX_DT = {1: ir.F32, 2: ir.U8, 3: ir.I8, 6: ir.I32, 7: ir.I64, 9: ir.BOOL, 10: ir.F16, 12: ir.U32, 21: ir.U4, 22: ir.I4}
_ONNX_DT_REV = {v: k for k, v in _ONNX_DT.items()}
_NP_OF = {ir.F32: np.float32, ir.F16: np.float16, ir.I64: np.int64, ir.I32: np.int32, ir.U32: np.uint32, ir.U8: np.uint8,
          ir.I8: np.int8, ir.BOOL: np.bool_}


class OnnxError(ValueError):
    pass


# ── protobuf wire format ─────────────────────────────────────────────────
def _varint(buf, i):
    shift = val = 0
    while True:
        b = buf[i]
        i += 1
        val |= (b & 0x7F) << shift
        if not b & 0x80:
            return val, i
        shift += 7


def _fields(buf):
    """Yields (field number, wire type, value) of one message; LEN fields as memoryview slices."""
    buf = memoryview(buf)
    i, n = 0, len(buf)
    while i < n:
        key, i = _varint(buf, i)
        field, wire = key >> 3, key & 7
        if wire == 0:
            v, i = _varint(buf, i)
        elif wire == 1:
            v, i = struct.unpack_from("<Q", buf, i)[0], i + 8
        elif wire == 2:
            ln, i = _varint(buf, i)
            v, i = buf[i:i + ln], i + ln
        elif wire == 5:
            v, i = struct.unpack_from("<I", buf, i)[0], i + 4
        else:
            raise OnnxError(f"unsupported protobuf wire type {wire}")
        yield field, wire, v


def _enc_varint(v: int) -> bytes:
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        out.append(b | (0x80 if v else 0))
        if not v:
            return bytes(out)


def _f_int(field, v):
    return _enc_varint(field << 3) + _enc_varint(v)


def _f_bytes(field, payload):
    payload = bytes(payload)
    return _enc_varint((field << 3) | 2) + _enc_varint(len(payload)) + payload


def _f_str(field, s):
    return _f_bytes(field, s.encode())


def _f_f32(field, v):
    return _enc_varint((field << 3) | 5) + struct.pack("<f", v)


def _signed(v):
    return v - (1 << 64) if v >= 1 << 63 else v


# ── reading ──────────────────────────────────────────────────────────────
class _Node:
    __slots__ = ("op", "domain", "name", "inputs", "outputs", "attrs")


def _parse_tensor(buf, external=None):
    """TensorProto → (name, dtype, dims, bytes). `external` resolves a tensor whose bytes live outside the model file
    (data_location = EXTERNAL with location / offset / length entries, parser.rs:297-380): a callable
    (location, offset, length or None) → uint8 array."""
    dims, dt, raw, name = [], 0, None, ""
    f32, i32, i64, u64, other_typed = [], [], [], [], False
    ext, ext_loc = {}, 0
    for f, w, v in _fields(buf):
        if f == 13:  # external_data: StringStringEntryProto {key = 1, value = 2}
            kv = {f2: bytes(v2).decode() for f2, _, v2 in _fields(v)}
            ext[kv.get(1, "")] = kv.get(2, "")
            continue
        if f == 14:  # data_location
            ext_loc = v
            continue
        if f == 1:
            if w == 2:  # packed
                j = 0
                while j < len(v):
                    d, j = _varint(v, j)
                    dims.append(d)
            else:
                dims.append(v)
        elif f == 2:
            dt = v
        elif f == 4:
            f32 += list(np.frombuffer(v, "<f4")) if w == 2 else [struct.unpack("<f", struct.pack("<I", v))[0]]
        elif f == 5:
            if w == 2:
                j = 0
                while j < len(v):
                    d, j = _varint(v, j)
                    i32.append(_signed(d))
            else:
                i32.append(_signed(v))
        elif f == 7:
            if w == 2:
                j = 0
                while j < len(v):
                    d, j = _varint(v, j)
                    i64.append(_signed(d))
            else:
                i64.append(_signed(v))
        elif f == 8:
            name = bytes(v).decode()
        elif f == 9:
            raw = bytes(v)
        elif f == 11:  # uint64_data
            if w == 2:
                j = 0
                while j < len(v):
                    d, j = _varint(v, j)
                    u64.append(d)
            else:
                u64.append(v)
        elif f in (6, 10):  # string_data, double_data
            other_typed = True
    if dt not in _ONNX_DT:
        raise OnnxError(f"initializer '{name}': unsupported ONNX data type {dt}")
    dtype = _ONNX_DT[dt]
    if ext_loc == 1:
        if external is None or "location" not in ext:
            raise OnnxError(f"initializer '{name}' keeps its data in an external file; load the model from its path")
        try:
            offset, length = int(ext.get("offset", "0")), (int(ext["length"]) if "length" in ext else None)
        except ValueError:
            raise OnnxError(f"initializer '{name}': invalid offset / length in external_data") from None
        return name, dtype, dims, external(ext["location"], offset, length)
    if raw is None:
        raw = _typed_to_raw(name, dtype, f32, i32, i64, u64, other_typed)
        if raw is None:
            if int(np.prod(dims)) if dims else 1:
                raise OnnxError(f"initializer '{name}' ({int(np.prod(dims)) if dims else 1} elements) carries no data: raw_data, "
                                "external data and the typed data fields are all empty")
            raw = b""
    return name, dtype, dims, np.frombuffer(raw, np.uint8).copy()


def _typed_to_raw(name, dtype, f32, i32, i64, u64, other_typed):
    """The typed data fields (the older encoding some exporters still write) as little-endian bytes, like raw_data;
    None when none is filled. int32_data carries every integer type below 32 bits, bool, and float16 as bit patterns
    (parser.rs:221-292). A filled field that does not match the declared type is an error, not an empty weight."""
    def mismatch(field):
        return OnnxError(f"initializer '{name}': {field} is populated but the declared data type is {ir.DTYPE_NAMES[dtype]}")
    if f32:
        if dtype != ir.F32:
            raise mismatch("float_data")
        return np.asarray(f32, "<f4").tobytes()
    if i64:
        if dtype != ir.I64:
            raise mismatch("int64_data")
        return np.asarray(i64, "<i8").tobytes()
    if i32:
        a = np.asarray(i32, np.int64)
        if dtype == ir.I32:
            return a.astype("<i4").tobytes()
        if dtype in (ir.U8, ir.I8):
            return (a & 0xFF).astype(np.uint8).tobytes()
        if dtype == ir.BOOL:
            return (a != 0).astype(np.uint8).tobytes()
        if dtype == ir.F16:
            return (a & 0xFFFF).astype("<u2").tobytes()  # bit patterns in the low 16 bits
        raise OnnxError(f"initializer '{name}': int32_data with data type {ir.DTYPE_NAMES[dtype]}")
    if u64:
        if dtype != ir.U32:
            raise mismatch("uint64_data")
        return (np.asarray(u64, np.uint64) & 0xFFFFFFFF).astype("<u4").tobytes()
    if other_typed:
        raise OnnxError(f"initializer '{name}': double / string typed data")
    return None


def _parse_attr(buf, external=None):
    name, out, ints, floats, typ = "", None, [], [], 0
    for f, w, v in _fields(buf):
        if f == 1:
            name = bytes(v).decode()
        elif f == 2:
            out = struct.unpack("<f", struct.pack("<I", v))[0]
        elif f == 3:
            out = _signed(v)
        elif f == 4:
            out = bytes(v).decode()
        elif f == 5:
            out = _parse_tensor(v, external)
        elif f == 7:
            floats += list(np.frombuffer(v, "<f4")) if w == 2 else [struct.unpack("<f", struct.pack("<I", v))[0]]
        elif f == 8:
            if w == 2:
                j = 0
                while j < len(v):
                    d, j = _varint(v, j)
                    ints.append(_signed(d))
            else:
                ints.append(_signed(v))
        elif f == 20:
            typ = v
    if typ == 7 or (out is None and ints):
        out = ints
    elif typ == 6 or (out is None and floats):
        out = [float(x) for x in floats]
    return name, out


def _parse_value_info(buf):
    name, elem, shape = "", 0, None
    for f, _, v in _fields(buf):
        if f == 1:
            name = bytes(v).decode()
        elif f == 2:  # TypeProto
            for f2, _, v2 in _fields(v):
                if f2 == 1:  # tensor_type
                    for f3, _, v3 in _fields(v2):
                        if f3 == 1:
                            elem = v3
                        elif f3 == 2:  # TensorShapeProto
                            shape = []
                            for f4, _, v4 in _fields(v3):
                                if f4 == 1:
                                    dim = None
                                    for f5, _, v5 in _fields(v4):
                                        if f5 == 1:
                                            dim = _signed(v5)
                                        elif f5 == 2:
                                            dim = bytes(v5).decode()
                                    shape.append(dim)
    return name, elem, shape


def parse_model(data: bytes, external=None):
    """ModelProto bytes → (nodes, initializers{name: (dtype, dims, bytes)}, inputs[(name, dtype, shape)], output names).
    `external`: see `_parse_tensor`."""
    graph = None
    for f, _, v in _fields(data):
        if f == 7:
            graph = v
    if graph is None:
        raise OnnxError("the model has no graph")
    nodes, inits, inputs, outputs = [], {}, [], []
    for f, _, v in _fields(graph):
        if f == 1:
            n = _Node()
            n.op, n.domain, n.name, n.inputs, n.outputs, n.attrs = "", "", "", [], [], {}
            for f2, _, v2 in _fields(v):
                if f2 == 1:
                    n.inputs.append(bytes(v2).decode())
                elif f2 == 2:
                    n.outputs.append(bytes(v2).decode())
                elif f2 == 3:
                    n.name = bytes(v2).decode()
                elif f2 == 4:
                    n.op = bytes(v2).decode()
                elif f2 == 5:
                    k, a = _parse_attr(v2, external)
                    n.attrs[k] = a
                elif f2 == 7:
                    n.domain = bytes(v2).decode()
            nodes.append(n)
        elif f == 5:
            name, dtype, dims, raw = _parse_tensor(v, external)
            inits[name] = (dtype, dims, raw)
        elif f == 11:
            inputs.append(_parse_value_info(v))
        elif f == 12:
            outputs.append(_parse_value_info(v)[0])
    return nodes, inits, inputs, outputs


# ── lowering ─────────────────────────────────────────────────────────────
class _Val:
    __slots__ = ("vid", "dtype", "shape", "content", "const")

    def __init__(self, vid, dtype, shape, content=None, const=None):
        self.vid, self.dtype, self.shape, self.content, self.const = vid, dtype, list(shape), content, const


class _Lower:
    def __init__(self, nodes, inits, inputs, outputs):
        self.b = ir.GraphBuilder()
        self.nodes, self.inits, self.outputs = nodes, inits, outputs
        self.vals: dict = {}
        self.syms: dict = {}
        self._fresh = 0
        for name, elem, shape in inputs:
            if name in inits:
                continue
            if elem not in _ONNX_DT or shape is None:
                raise OnnxError(f"input '{name}' needs a tensor type with a shape")
            dims = [self._dim(d) for d in shape]
            self.vals[name] = _Val(self.b.input(name, _ONNX_DT[elem], dims), _ONNX_DT[elem], dims)

    def _dim(self, d):
        if isinstance(d, str):
            if d not in self.syms:
                self.syms[d] = self.b.sym(d)
            return self.syms[d]
        if d is None:  # neither a value nor a name: the symbol "unknown", as the reference names it (parser.rs:619-622)
            return self._dim("unknown")
        if d < 0:
            raise OnnxError("negative input dimension")
        return DimExpr.of(d)

    # operands ----------------------------------------------------------
    def has(self, node, i):
        return i < len(node.inputs) and node.inputs[i] != ""

    def const_array(self, name):
        """Value of an initializer as a numpy array (for operands that must be compile-time constants)."""
        if name in self.vals and self.vals[name].const is not None:
            return self.vals[name].const
        if name not in self.inits:
            return None
        dtype, dims, raw = self.inits[name]
        if dtype not in _NP_OF:
            return None
        return raw.view(_NP_OF[dtype]).reshape(dims)

    def val(self, name, as_type=None):
        """Operand by name; an initializer becomes a module constant on first use. `as_type` = (dtype, dims)
        reinterprets the initializer's bytes (packed nibbles shipped as uint8)."""
        if name in self.vals and as_type is None:
            return self.vals[name]
        if name not in self.inits:
            if name in self.vals:
                raise OnnxError(f"'{name}' must be an initializer to be reinterpreted")
            raise OnnxError(f"operand '{name}' is not defined")
        dtype, dims, raw = self.inits[name]
        if as_type is not None:
            dtype, dims = as_type
            if ir.storage_bytes(dtype, int(np.prod(dims))) != raw.size:
                raise OnnxError(f"initializer '{name}' has {raw.size} bytes, not what {ir.DTYPE_NAMES[dtype]}{list(dims)} needs")
        t = HostTensor(dtype, list(dims), raw)
        v = _Val(self.b.constant(t, borrow=raw.size > 1 << 16), dtype, [DimExpr.of(d) for d in dims],
                 const=self.const_array(name) if as_type is None else None)
        if as_type is None:
            self.vals[name] = v
        return v

    def int_list(self, node, i, attr=None):
        """A list of integers given as a constant operand (newer opsets) or an attribute (older ones)."""
        if self.has(node, i):
            a = self.const_array(node.inputs[i])
            if a is None:
                raise OnnxError(f"{node.op} '{node.name}': operand {i} must be a constant")
            return [int(x) for x in np.asarray(a).reshape(-1)]
        if attr is not None and attr in node.attrs:
            return [int(x) for x in node.attrs[attr]]
        return None

    def set(self, node, i, val):
        if i < len(node.outputs) and node.outputs[i]:
            self.vals[node.outputs[i]] = val

    def vid(self, v):
        """The module value of an operand; a compile-time shape value consumed by a tensor operation is
        materialised as a DimValues node evaluated at run time (lib.rs value(): Content → DimValues)."""
        if v.vid is None:
            out = self.b.dim_values(list(v.content))
            if not v.shape:
                out = self.b.reshape(out, [])
            if v.dtype != ir.I64:
                out = self.b.cast(out, v.dtype)
            v.vid = out
        return v.vid

    def content_of(self, name):
        """Compile-time integer content of an operand: a shape value, or a small integer initializer. None otherwise."""
        v = self.val(name)
        if v.content is not None:
            return list(v.content)
        if v.const is not None and v.dtype in (ir.I64, ir.I32) and v.const.ndim <= 1 and v.const.size <= 64:
            return [int(c) for c in np.asarray(v.const).reshape(-1)]
        return None

    @staticmethod
    def _signed_const(d):
        """A dimension expression or an integer as a Python int when it has no symbols (negative values included)."""
        if isinstance(d, DimExpr):
            if not d.terms:
                return 0
            return d.terms[()] if list(d.terms) == [()] else None
        return int(d)

    @staticmethod
    def _div_exact(d, k):
        d = DimExpr.of(d)
        if k == 0 or any(c % k for c in d.terms.values()):
            return None
        return DimExpr({s: c // k for s, c in d.terms.items()})

    @staticmethod
    def _broadcast(a, b):
        ra, rb = list(a), list(b)
        while len(ra) < len(rb):
            ra.insert(0, DimExpr.of(1))
        while len(rb) < len(ra):
            rb.insert(0, DimExpr.of(1))
        return [y if x == 1 else x for x, y in zip(ra, rb)]

    # rules -------------------------------------------------------------
    def lower(self):
        for node in self.nodes:
            self.b.set_loc(node.name or None, node.op)
            rule = getattr(self, "op_" + node.op.replace(".", "_"), None)
            if rule is None:
                raise OnnxError(f"no lowering rule for operator '{node.op}'" + (f" (domain {node.domain})" if node.domain else ""))
            rule(node)
        self.b.set_loc(None)
        self._finish_outputs()
        m = self.b.finish()
        m.fold_transposes()  # MatMul(h, Transpose(W)) of tied-embedding exports (fold.rs:129-178)
        return m

    def _finish_outputs(self):
        for name in self.outputs:
            if name not in self.vals and name not in self.inits:
                raise OnnxError(f"graph output '{name}' was never produced")
            v = self.val(name)
            if v.vid is None:
                # a shape value whose elements are all constants leaves as an i64 constant; a symbolic one cannot (lib.rs:513-523)
                vals = [self._signed_const(c) for c in v.content]
                if None in vals:
                    raise OnnxError(f"graph output '{name}' is a symbolic shape value")
                dims = [d.as_const() for d in v.shape]
                self.b.output(name, self.b.const_i64(vals, dims))
                continue
            self.b.output(name, v.vid)

    def op_Identity(self, n):
        self.set(n, 0, self.val(n.inputs[0]))

    def _binary(self, n, op, out_dtype=None):
        a, b = self.val(n.inputs[0]), self.val(n.inputs[1])
        if op in (ir.ADD, ir.SUB, ir.MUL, ir.DIV) and (a.content is not None or b.content is not None):
            ca, cb = self.content_of(n.inputs[0]), self.content_of(n.inputs[1])
            if ca is not None and cb is not None and (len(ca) == len(cb) or 1 in (len(ca), len(cb))):
                m = max(len(ca), len(cb))
                ca, cb = ca * (m // len(ca)), cb * (m // len(cb))
                f = {ir.ADD: lambda x, y: DimExpr.of(x) + y, ir.SUB: lambda x, y: DimExpr.of(x) - y, ir.MUL: lambda x, y: DimExpr.of(x) * y,
                     ir.DIV: lambda x, y: self._div_exact(x, self._signed_const(y) or 0)}[op]
                out = [f(x, y) for x, y in zip(ca, cb)]
                if None not in out:
                    shape = a.shape if len(a.shape) >= len(b.shape) else b.shape
                    self.set(n, 0, _Val(None, a.dtype, shape, content=out))
                    return
        self.set(n, 0, _Val(self.b.binary(op, self.vid(a), self.vid(b)), out_dtype or a.dtype, self._broadcast(a.shape, b.shape)))

    def op_Add(self, n): self._binary(n, ir.ADD)
    def op_Sub(self, n): self._binary(n, ir.SUB)
    def op_Mul(self, n): self._binary(n, ir.MUL)
    def op_Div(self, n): self._binary(n, ir.DIV)
    def op_And(self, n): self._binary(n, ir.AND)
    def op_Or(self, n): self._binary(n, ir.OR)
    def op_Xor(self, n): self._binary(n, ir.XOR)

    def op_Pow(self, n):
        # ONNX lets the exponent have another type; the primitive wants the base's (rules.rs:116-125)
        a, b = self.val(n.inputs[0]), self.val(n.inputs[1])
        bv = self.vid(b) if b.dtype == a.dtype else self.b.cast(self.vid(b), a.dtype)
        self.set(n, 0, _Val(self.b.binary(ir.POW, self.vid(a), bv), a.dtype, self._broadcast(a.shape, b.shape)))

    def _variadic(self, n, op):
        # Max / Min take any number of operands: folded from the left (rules.rs:127-136)
        acc = self.val(n.inputs[0])
        out, shape = self.vid(acc), list(acc.shape)
        for name in n.inputs[1:]:
            r = self.val(name)
            out, shape = self.b.binary(op, out, self.vid(r)), self._broadcast(shape, r.shape)
        self.set(n, 0, _Val(out, acc.dtype, shape))

    def op_Max(self, n): self._variadic(n, ir.MAX)
    def op_Min(self, n): self._variadic(n, ir.MIN)

    def _compare(self, n, op):
        a, b = self.val(n.inputs[0]), self.val(n.inputs[1])
        self.set(n, 0, _Val(self.b.cmp(op, self.vid(a), self.vid(b)), ir.BOOL, self._broadcast(a.shape, b.shape)))

    def op_Equal(self, n): self._compare(n, ir.EQ)
    def op_Greater(self, n): self._compare(n, ir.GT)
    def op_GreaterOrEqual(self, n): self._compare(n, ir.GE)
    def op_Less(self, n): self._compare(n, ir.LT)
    def op_LessOrEqual(self, n): self._compare(n, ir.LE)

    def _unary(self, n, op):
        x = self.val(n.inputs[0])
        self.set(n, 0, _Val(self.b.unary(op, self.vid(x)), x.dtype, x.shape))

    def op_Neg(self, n): self._unary(n, ir.NEG)
    def op_Abs(self, n): self._unary(n, ir.ABS)
    def op_Sqrt(self, n): self._unary(n, ir.SQRT)
    def op_Exp(self, n): self._unary(n, ir.EXP)
    def op_Log(self, n): self._unary(n, ir.LOG)
    def op_Sin(self, n): self._unary(n, ir.SIN)
    def op_Cos(self, n): self._unary(n, ir.COS)
    def op_Tanh(self, n): self._unary(n, ir.TANH)
    def op_Erf(self, n): self._unary(n, ir.ERF)
    def op_Floor(self, n): self._unary(n, ir.FLOOR)
    def op_Ceil(self, n): self._unary(n, ir.CEIL)
    def op_Not(self, n): self._unary(n, ir.NOT)

    def op_Where(self, n):
        c, a, b = (self.val(i) for i in n.inputs[:3])
        shape = self._broadcast(self._broadcast(c.shape, a.shape), b.shape)
        self.set(n, 0, _Val(self.b.select(self.vid(c), self.vid(a), self.vid(b)), a.dtype, shape))

    def op_Constant(self, n):
        """A Constant node is an initializer spelled as a node (parser.rs:81-100)."""
        a = n.attrs
        if "value" in a:
            _, dtype, dims, raw = a["value"]
        elif "value_int" in a or "value_ints" in a:
            arr = np.asarray(a.get("value_ints", a.get("value_int")), np.int64)
            dtype, dims, raw = ir.I64, list(arr.shape), np.frombuffer(arr.tobytes(), np.uint8).copy()
        elif "value_float" in a or "value_floats" in a:
            arr = np.asarray(a.get("value_floats", a.get("value_float")), np.float32)
            dtype, dims, raw = ir.F32, list(arr.shape), np.frombuffer(arr.tobytes(), np.uint8).copy()
        else:
            raise OnnxError(f"Constant '{n.name}' carries no tensor, integer or float value")
        self.inits[n.outputs[0]] = (dtype, list(dims), raw)

    def op_Cast(self, n):
        x = self.val(n.inputs[0])
        to = _ONNX_DT.get(n.attrs.get("to"))
        if to is None:
            raise OnnxError(f"Cast '{n.name}': unsupported target type {n.attrs.get('to')}")
        if x.content is not None:  # shape values stay shape values whatever integer type they are cast to
            self.set(n, 0, _Val(None, to, x.shape, content=x.content))
        else:
            self.set(n, 0, _Val(self.b.cast(x.vid, to), to, x.shape))

    def op_Shape(self, n):
        """The operand's dimensions as a compile-time value, never a tensor; `start` / `end` (negative from the end,
        clamped to the rank) select a range (rules.rs:536-563)."""
        x = self.val(n.inputs[0])
        dims = list(x.shape) if x.content is None else [DimExpr.of(len(x.content))]
        rank = len(dims)

        def bound(v):
            v = v + rank if v < 0 else v
            return max(0, min(rank, v))
        start, end = bound(int(n.attrs.get("start", 0))), bound(int(n.attrs.get("end", rank)))
        picked = dims[min(start, end):end]
        self.set(n, 0, _Val(None, ir.I64, [DimExpr.of(len(picked))], content=picked))

    def op_Gather(self, n):
        data, axis = self.val(n.inputs[0]), int(n.attrs.get("axis", 0))
        if data.content is not None:
            idx = self.const_array(n.inputs[1])
            if idx is None:
                raise OnnxError(f"Gather '{n.name}' on a shape value needs constant indices")
            picks = [data.content[int(i)] for i in np.asarray(idx).reshape(-1)]
            self.set(n, 0, _Val(None, data.dtype, [] if np.asarray(idx).ndim == 0 else [DimExpr.of(len(picks))], content=picks))
            return
        idx = self.val(n.inputs[1])
        if axis < 0:
            axis += len(data.shape)
        ivid = self.vid(idx) if idx.dtype == ir.I64 else self.b.cast(self.vid(idx), ir.I64)  # the primitive takes i64 indices (rules.rs:503-522)
        shape = data.shape[:axis] + idx.shape + data.shape[axis + 1:]
        self.set(n, 0, _Val(self.b.gather(data.vid, ivid, axis), data.dtype, shape))

    def _reduce(self, n, op):
        x = self.val(n.inputs[0])
        axes = self.int_list(n, 1, "axes")
        keep = bool(n.attrs.get("keepdims", 1))
        if x.content is not None and axes in (None, [0], [-1]) and op in (ir.SUM, ir.PROD):
            acc = DimExpr.of(0 if op == ir.SUM else 1)  # e.g. ReduceProd over a shape vector = element count
            for c in x.content:
                acc = acc + c if op == ir.SUM else acc * c
            self.set(n, 0, _Val(None, x.dtype, [DimExpr.of(1)] if keep else [], content=[acc]))
            return
        if not axes:
            if int(n.attrs.get("noop_with_empty_axes", 0)):
                self.set(n, 0, x)
                return
            axes = list(range(len(x.shape)))
        axes = sorted({self._axis(n, a, len(x.shape)) for a in axes})
        shape = [DimExpr.of(1) if i in axes else d for i, d in enumerate(x.shape) if keep or i not in axes]
        self.set(n, 0, _Val(self.b.reduce(op, self.vid(x), axes, keep), x.dtype, shape))

    def op_ReduceSum(self, n): self._reduce(n, ir.SUM)
    def op_ReduceMean(self, n): self._reduce(n, ir.MEAN)
    def op_ReduceMax(self, n): self._reduce(n, ir.RMAX)
    def op_ReduceMin(self, n): self._reduce(n, ir.RMIN)
    def op_ReduceProd(self, n): self._reduce(n, ir.PROD)

    def _axis(self, n, a, rank):
        if not -rank <= a < max(rank, 1):
            raise OnnxError(f"{n.op} '{n.name}': axis {a} is outside rank {rank}")
        return a + rank if a < 0 else a

    def op_Slice(self, n):
        """Bounds may be shape arithmetic; axes and steps are constants (rules.rs:421-501). An end of INT32_MAX or
        more means "to the end", negative constants count from the end, constants are clamped to constant extents."""
        x = self.val(n.inputs[0])
        starts = self.content_of(n.inputs[1]) if self.has(n, 1) else n.attrs.get("starts")
        ends = self.content_of(n.inputs[2]) if self.has(n, 2) else n.attrs.get("ends")
        if starts is None or ends is None:
            raise OnnxError(f"Slice '{n.name}': starts / ends are not resolvable when the graph is lowered")
        dims = [DimExpr.of(len(x.content))] if x.content is not None else list(x.shape)
        axes = self.int_list(n, 3, "axes") or list(range(len(starts)))
        steps = self.int_list(n, 4) or [1] * len(starts)
        specs, shape = [], list(dims)
        for s, e, ax, st in zip(starts, ends, axes, steps):
            ax = self._axis(n, ax, len(dims))
            dim = dims[ax]

            def norm(bound, is_end):
                v = self._signed_const(bound)
                if v is None:
                    return DimExpr.of(bound)
                if is_end and v >= (1 << 31) - 1:
                    return dim
                if v < 0:
                    return dim + v
                return DimExpr.of(min(v, dim.as_const()) if dim.as_const() is not None else v)
            lo, hi = norm(s, False), norm(e, True)
            if st == 1:
                shape[ax] = hi - lo
            elif st == -1:
                shape[ax] = lo - hi
            else:
                a, b = self._signed_const(lo), self._signed_const(hi)
                if st == 0 or a is None or b is None:
                    raise OnnxError(f"Slice '{n.name}': step {st} needs constant bounds")
                shape[ax] = DimExpr.of(max(0, -(-(b - a) // st) if st > 0 else -(-(a - b) // -st)))
            specs.append((ax, lo, hi, int(st)))
        if x.content is not None:  # a piece of a shape vector
            (ax, lo, hi, st), = specs
            a, b = self._signed_const(lo), self._signed_const(hi)
            self.set(n, 0, _Val(None, x.dtype, [DimExpr.of(len(x.content[a:b:st]))], content=x.content[a:b:st]))
            return
        self.set(n, 0, _Val(self.b.slice(x.vid, specs), x.dtype, shape))

    def op_Transpose(self, n):
        x = self.val(n.inputs[0])
        perm = [int(p) for p in n.attrs.get("perm", list(range(len(x.shape)))[::-1])]
        self.set(n, 0, _Val(self.b.transpose(self.vid(x), perm), x.dtype, [x.shape[p] for p in perm]))

    def op_MatMul(self, n):
        # rank-1 operands are promoted in lowering, not in the primitive (rules.rs:171-213)
        a, b = self.val(n.inputs[0]), self.val(n.inputs[1])
        av, ash, bv, bsh = self.vid(a), list(a.shape), self.vid(b), list(b.shape)
        if len(ash) == 1:
            ash = [DimExpr.of(1)] + ash
            av = self.b.reshape(av, ash)
        if len(bsh) == 1:
            bsh = bsh + [DimExpr.of(1)]
            bv = self.b.reshape(bv, bsh)
        out = self.b.matmul(av, bv)
        shape = self._broadcast(ash[:-2], bsh[:-2]) + [ash[-2], bsh[-1]]
        if len(a.shape) == 1:
            shape = shape[:-2] + shape[-1:]
        if len(b.shape) == 1:
            shape = shape[:-1]
        if len(a.shape) == 1 or len(b.shape) == 1:
            out = self.b.reshape(out, shape)
        self.set(n, 0, _Val(out, a.dtype, shape))

    def op_Reshape(self, n):
        x = self.val(n.inputs[0])
        tgt = self.val(n.inputs[1])
        if tgt.content is not None:
            dims = list(tgt.content)
        else:
            arr = self.const_array(n.inputs[1])
            if arr is None:
                raise OnnxError(f"Reshape '{n.name}': the target shape must be a constant or shape arithmetic")
            dims = [int(v) for v in np.asarray(arr).reshape(-1)]
        out, unknown = [], -1
        for i, d in enumerate(dims):
            if isinstance(d, DimExpr) and self._signed_const(d) is not None:
                d = self._signed_const(d)  # a constant that came through shape arithmetic
            if isinstance(d, DimExpr):
                out.append(d)
            elif d == 0 and not int(n.attrs.get("allowzero", 0)):
                out.append(x.shape[i])  # 0 copies the input's dimension
            elif d == -1:
                if unknown >= 0:
                    raise OnnxError(f"Reshape '{n.name}' allows at most one -1")
                unknown = i
                out.append(None)
            elif d < 0:
                raise OnnxError(f"Reshape '{n.name}': invalid dimension {d}")
            else:
                out.append(DimExpr.of(d))
        if unknown >= 0:
            # the one free dimension: the element count divided by the known extents when that is exact, otherwise a
            # fresh symbol that is bound from the element count when the graph runs (rules.rs:247-259)
            numel, known = DimExpr.of(1), DimExpr.of(1)
            for d in x.shape:
                numel = numel * d
            for j, d in enumerate(out):
                if j != unknown:
                    known = known * d
            inferred = numel.div_exact(known)
            if inferred is None:
                self._fresh += 1
                inferred = self.b.sym(f"reshape#{self._fresh}")
            out[unknown] = inferred
        self.set(n, 0, _Val(self.b.reshape(self.vid(x), out), x.dtype, out))

    def op_Unsqueeze(self, n):
        x = self.val(n.inputs[0])
        axes = self.int_list(n, 1, "axes")
        rank = len(x.shape) + len(axes)
        axes = sorted(a + rank if a < 0 else a for a in axes)
        if x.content is not None:  # shape arithmetic: a scalar becomes a one-element vector
            self.set(n, 0, _Val(None, x.dtype, [DimExpr.of(len(x.content))], content=list(x.content)))
            return
        shape, it = [], iter(x.shape)
        for i in range(rank):
            shape.append(DimExpr.of(1) if i in axes else next(it))
        self.set(n, 0, _Val(self.b.reshape(x.vid, shape), x.dtype, shape))

    def op_Concat(self, n):
        vals = [self.val(i) for i in n.inputs]
        axis = int(n.attrs.get("axis", 0))
        if all(v.content is not None or v.const is not None for v in vals) and any(v.content is not None for v in vals):
            content = []
            for v in vals:  # shape arithmetic: pieces of a target shape
                content += list(v.content) if v.content is not None else [int(c) for c in np.asarray(v.const).reshape(-1)]
            self.set(n, 0, _Val(None, ir.I64, [DimExpr.of(len(content))], content=content))
            return
        axis = axis + len(vals[0].shape) if axis < 0 else axis
        shape = list(vals[0].shape)
        for v in vals[1:]:
            shape[axis] = shape[axis] + v.shape[axis]
        self.set(n, 0, _Val(self.b.concat([self.vid(v) for v in vals], axis), vals[0].dtype, shape))

    def op_Squeeze(self, n):
        x = self.val(n.inputs[0])
        axes = self.int_list(n, 1, "axes")
        if x.content is not None:  # a one-element shape vector becomes a scalar shape value
            self.set(n, 0, _Val(None, x.dtype, [], content=list(x.content)))
            return
        drop = ([self._axis(n, a, len(x.shape)) for a in axes] if axes is not None
                else [i for i, d in enumerate(x.shape) if d.as_const() == 1])
        shape = [d for i, d in enumerate(x.shape) if i not in drop]
        self.set(n, 0, _Val(self.b.reshape(x.vid, shape), x.dtype, shape))

    def op_Expand(self, n):
        x = self.val(n.inputs[0])
        target = self.content_of(n.inputs[1])
        if target is None:
            raise OnnxError(f"Expand '{n.name}': the shape is not resolvable when the graph is lowered")
        shape = self._broadcast(x.shape, [DimExpr.of(d) for d in target])  # ONNX Expand broadcasts both ways
        self.set(n, 0, _Val(self.b.broadcast(self.vid(x), shape), x.dtype, shape))

    def op_ScatterND(self, n):
        if n.attrs.get("reduction", "none") != "none":
            raise OnnxError(f"ScatterND reduction='{n.attrs['reduction']}'")
        data, idx, upd = (self.val(i) for i in n.inputs[:3])
        ivid = self.vid(idx) if idx.dtype == ir.I64 else self.b.cast(self.vid(idx), ir.I64)
        self.set(n, 0, _Val(self.b.scatter(self.vid(data), ivid, self.vid(upd)), data.dtype, data.shape))

    def op_Range(self, n):
        """Iota plus element-wise arithmetic; start and delta are constants, the limit may be a shape value
        (rules.rs:566-606)."""
        parts = []
        for i in range(3):
            v = self.val(n.inputs[i])
            c = self.content_of(n.inputs[i])
            if c is None and v.const is not None and v.const.size == 1 and v.dtype in (ir.I64, ir.I32):
                c = [int(np.asarray(v.const).reshape(-1)[0])]
            if not c:
                raise OnnxError(f"Range '{n.name}': bounds are not resolvable when the graph is lowered")
            parts.append(c[0])
        start, delta = self._signed_const(parts[0]), self._signed_const(parts[2])
        if start is None or delta is None:
            raise OnnxError(f"Range '{n.name}' with a symbolic start or delta")
        if delta <= 0:
            raise OnnxError(f"Range with delta {delta}")
        length = self._div_exact(DimExpr.of(parts[1]) - start, delta)
        if length is None:
            raise OnnxError(f"Range '{n.name}': the length is not exactly divisible by delta")
        dtype = self.val(n.inputs[0]).dtype
        out = self.b.iota(length, ir.I64)
        if delta != 1:
            out = self.b.mul(out, self.b.const_i64([delta], []))
        if start != 0:
            out = self.b.add(out, self.b.const_i64([start], []))
        if dtype != ir.I64:
            out = self.b.cast(out, dtype)
        self.set(n, 0, _Val(out, dtype, [length]))

    def op_ConstantOfShape(self, n):
        target = self.content_of(n.inputs[0])
        if target is None:
            raise OnnxError(f"ConstantOfShape '{n.name}': the shape is not resolvable when the graph is lowered")
        if "value" in n.attrs:
            _, dtype, _, raw = n.attrs["value"]
        else:  # the operator's default fill: one f32 zero
            dtype, raw = ir.F32, np.zeros(4, np.uint8)
        scalar = self.b.constant(HostTensor(dtype, [], raw))
        shape = [DimExpr.of(d) for d in target]
        self.set(n, 0, _Val(self.b.broadcast(scalar, shape), dtype, shape))

    def op_Trilu(self, n):
        x = self.val(n.inputs[0])
        k = 0
        if self.has(n, 1):
            ks = self.int_list(n, 1)
            k = ks[0] if ks else 0
        out = self.b.composite("Trilu", {"upper": int(n.attrs.get("upper", 1)), "k": int(k)}, [self.vid(x)], [(x.dtype, x.shape)])
        self.set(n, 0, _Val(out[0], x.dtype, x.shape))

    def _rotary(self, n, name):
        ins = [self.val(n.inputs[i]) for i in range(4)]  # input, position_ids, cos_cache, sin_cache
        attrs = {"interleaved": int(n.attrs.get("interleaved", 0)), "num_heads": max(int(n.attrs.get("num_heads", 0)), 0),
                 "rotary_embedding_dim": int(n.attrs.get("rotary_embedding_dim", 0))}
        x = ins[0]
        out = self.b.composite(name, attrs, [self.vid(v) for v in ins], [(x.dtype, x.shape)])
        self.set(n, 0, _Val(out[0], x.dtype, x.shape))

    def op_RotaryEmbedding(self, n): self._rotary(n, "com.microsoft.RotaryEmbedding")
    def op_GemmaRotaryEmbedding(self, n): self._rotary(n, "com.microsoft.GemmaRotaryEmbedding")

    def op_SimplifiedLayerNormalization(self, n):
        x, w = self.val(n.inputs[0]), self.val(n.inputs[1])
        attrs = {"epsilon": float(n.attrs.get("epsilon", 1e-5)), "axis": int(n.attrs.get("axis", -1))}
        out = self.b.composite("SimplifiedLayerNormalization", attrs, [x.vid, w.vid], [(x.dtype, x.shape)])
        self.set(n, 0, _Val(out[0], x.dtype, x.shape))

    def op_Gelu(self, n):
        x = self.val(n.inputs[0])
        approx = n.attrs.get("approximate", "none")
        out = self.b.composite("Gelu", {"approximate": approx}, [x.vid], [(x.dtype, x.shape)])
        self.set(n, 0, _Val(out[0], x.dtype, x.shape))

    def op_FastGelu(self, n):  # com.microsoft: the tanh form
        n.attrs["approximate"] = "tanh"
        self.op_Gelu(n)

    def op_Softmax(self, n):
        x = self.val(n.inputs[0])
        axis = int(n.attrs.get("axis", -1))
        out = self.b.composite("Softmax", {"axis": axis + len(x.shape) if axis < 0 else axis}, [x.vid], [(x.dtype, x.shape)])
        self.set(n, 0, _Val(out[0], x.dtype, x.shape))

    def op_MatMulNBits(self, n):
        bits = int(n.attrs.get("bits", 4))
        if bits != 4:
            raise OnnxError(f"MatMulNBits bits={bits}")
        for a in ("K", "N", "block_size"):
            if a not in n.attrs:
                raise OnnxError(f"MatMulNBits '{n.name}': attribute '{a}' is missing")
        k, nn, bs = int(n.attrs["K"]), int(n.attrs["N"]), int(n.attrs["block_size"])
        nb = -(-k // bs)
        a = self.val(n.inputs[0])
        w = self.val(n.inputs[1], as_type=(ir.U4, [nn, nb, bs]))  # same bytes, honest logical type
        s = self.val(n.inputs[2])
        ins = [a.vid, w.vid, s.vid]
        if self.has(n, 3):
            try:
                ins.append(self.val(n.inputs[3], as_type=(ir.U4, [nn, nb])).vid)
            except OnnxError as e:
                raise OnnxError(f"MatMulNBits zero_points layout not reinterpretable (odd block counts are padded per row): {e}") from None
        shape = a.shape[:-1] + [DimExpr.of(nn)]
        out = self.b.composite("com.microsoft.MatMulNBits", {"K": k, "N": nn, "bits": bits, "block_size": bs}, ins, [(a.dtype, shape)])
        self.set(n, 0, _Val(out[0], a.dtype, shape))

    def op_GroupQueryAttention(self, n):
        if float(n.attrs.get("softcap", 0.0)) != 0.0:
            raise OnnxError("GroupQueryAttention with softcap")
        rot = int(n.attrs.get("do_rotary", 0)) != 0
        if rot and self.has(n, 9):
            raise OnnxError("GroupQueryAttention with do_rotary=1 and explicit position_ids")
        if len(n.inputs) < 7 or not all(self.has(n, i) for i in range(7)):
            raise OnnxError("GroupQueryAttention requires q/k/v, past KV, seqlens_k and total_sequence_length inputs")
        vals = [self.val(n.inputs[i]) for i in range(6)]
        if vals[5].dtype != ir.I32:
            raise OnnxError(f"GroupQueryAttention seqlens_k must be int32, got {ir.DTYPE_NAMES[vals[5].dtype]}")
        ins = [v.vid for v in vals]
        if rot:
            if not (self.has(n, 7) and self.has(n, 8)):
                raise OnnxError("GroupQueryAttention with do_rotary=1 requires cos/sin caches")
            ins += [self.val(n.inputs[7]).vid, self.val(n.inputs[8]).vid]
        bias = len(n.inputs) > 10 and self.has(n, 10)
        if bias:
            ins.append(self.val(n.inputs[10]).vid)
        for a in ("num_heads", "kv_num_heads"):
            if a not in n.attrs:
                raise OnnxError(f"GroupQueryAttention '{n.name}': attribute '{a}' is missing")
        attrs = {"num_heads": int(n.attrs["num_heads"]), "kv_num_heads": int(n.attrs["kv_num_heads"]),
                 "scale": float(n.attrs.get("scale", 0.0)), "local_window_size": int(n.attrs.get("local_window_size", -1)),
                 "do_rotary": int(rot), "rotary_interleaved": int(n.attrs.get("rotary_interleaved", 0)), "has_attention_bias": int(bias)}
        q, past = vals[0], vals[3]
        seq, p_rows = q.shape[1], past.shape[2]
        total = self.val(n.inputs[6])
        if total.content:  # computed from shapes by the export: a bind-time constraint, not an operand
            self.b.constrain(total.content[0], p_rows + seq,
                             "GroupQueryAttention 'total_sequence_length' must equal the past KV length plus the new sequence length")
        present = list(past.shape)
        present[2] = p_rows + seq
        outs = self.b.composite("com.microsoft.GroupQueryAttention", attrs, ins,
                                [(q.dtype, q.shape), (past.dtype, present), (past.dtype, present)])
        for i, o in enumerate(outs):
            self.set(n, i, _Val(o, q.dtype if i == 0 else past.dtype, q.shape if i == 0 else present))


def load_onnx_bytes(data: bytes, external_buffers: dict | None = None) -> ir.Module:
    """Model bytes → module. `external_buffers` maps the `location` of external tensor data to its bytes (the form the
    reference uses where there is no file system, parser.rs:297-330)."""
    resolver = None
    if external_buffers is not None:
        def resolver(location, offset, length):
            if location not in external_buffers:
                raise OnnxError(f"external data '{location}' was not provided")
            buf = np.frombuffer(external_buffers[location], np.uint8)
            end = len(buf) if length is None else offset + length
            if offset < 0 or end > len(buf):
                raise OnnxError(f"external data '{location}': bytes {offset}..{end} lie outside the buffer")
            return buf[offset:end].copy()
    return _Lower(*parse_model(data, resolver)).lower()


def load_onnx(path: str) -> ir.Module:
    """Model file → module; tensors with external data are read from the files beside it (memory-mapped, copied per tensor)."""
    import os
    base = os.path.dirname(os.path.abspath(path))
    maps: dict = {}

    def resolver(location, offset, length):
        full = os.path.normpath(os.path.join(base, location))
        if not full.startswith(base + os.sep):
            raise OnnxError(f"external data location '{location}' leaves the model's directory")
        if full not in maps:
            if not os.path.isfile(full):
                raise OnnxError(f"external data file '{location}' not found beside the model")
            maps[full] = np.memmap(full, np.uint8, "r")
        buf = maps[full]
        end = len(buf) if length is None else offset + length
        if offset < 0 or end > len(buf):
            raise OnnxError(f"external data '{location}': bytes {offset}..{end} lie outside the file")
        return np.array(buf[offset:end])

    with open(path, "rb") as f:
        return _Lower(*parse_model(f.read(), resolver)).lower()


# ── writing ──────────────────────────────────────────────────────────────
def _tensor_proto(name, arr, onnx_dtype=None, dims=None, external=None):
    """`external` = (location, offset): the bytes are not embedded; the caller writes them to that file at that offset."""
    arr = np.ascontiguousarray(arr)
    dt = onnx_dtype if onnx_dtype is not None else _ONNX_DT_REV[{np.dtype(v): k for k, v in _NP_OF.items()}[arr.dtype]]
    out = b"".join(_f_int(1, d) for d in (dims if dims is not None else arr.shape))
    out += _f_int(2, dt) + _f_str(8, name)
    if external is None:
        return out + _f_bytes(9, arr.tobytes())
    entries = (("location", external[0]), ("offset", str(external[1])), ("length", str(arr.nbytes)))
    return out + b"".join(_f_bytes(13, _f_str(1, k) + _f_str(2, v)) for k, v in entries) + _f_int(14, 1)


def _attr_proto(name, v):
    out = _f_str(1, name)
    if isinstance(v, bool) or isinstance(v, (int, np.integer)):
        return out + _f_int(3, int(v)) + _f_int(20, 2)
    if isinstance(v, float):
        return out + _f_f32(2, v) + _f_int(20, 1)
    if isinstance(v, str):
        return out + _f_bytes(4, v.encode()) + _f_int(20, 3)
    if isinstance(v, (list, tuple)):
        return out + b"".join(_f_int(8, int(x)) for x in v) + _f_int(20, 7)
    if isinstance(v, np.ndarray):  # an attribute tensor (ConstantOfShape 'value', Constant 'value')
        return out + _f_bytes(5, _tensor_proto("", v)) + _f_int(20, 4)
    raise OnnxError(f"attribute '{name}': unsupported value {v!r}")


def _value_info(name, dtype, shape):
    dims = b"".join(_f_bytes(1, _f_str(2, d) if isinstance(d, str) else _f_int(1, d)) for d in shape)
    tensor = _f_int(1, _ONNX_DT_REV[dtype]) + _f_bytes(2, dims)
    return _f_str(1, name) + _f_bytes(2, _f_bytes(1, tensor))


class OnnxWriter:
    """Collects nodes, initializers and the signature of one graph; `tobytes()` gives a ModelProto."""

    def __init__(self, name="graph"):
        self.name, self.nodes, self.inits, self.inputs, self.outputs = name, [], [], [], []
        self.external: dict = {}  # location → bytes of the initializers written as external data

    def node(self, op, inputs, outputs, name="", domain="", **attrs):
        body = b"".join(_f_str(1, i) for i in inputs) + b"".join(_f_str(2, o) for o in outputs)
        body += _f_str(3, name) + _f_str(4, op) + b"".join(_f_bytes(5, _attr_proto(k, v)) for k, v in attrs.items())
        if domain:
            body += _f_str(7, domain)
        self.nodes.append(body)
        return outputs[0]

    def initializer(self, name, arr, onnx_dtype=None, dims=None, external=None):
        """`external`: a location (file name beside the model); the bytes are appended to `self.external[location]`."""
        if external is not None:
            blob = self.external.setdefault(external, bytearray())
            blob.extend(b"\0" * (-len(blob) % 64))  # tensors start on 64-byte boundaries, as exporters write them
            self.inits.append(_tensor_proto(name, arr, onnx_dtype, dims, external=(external, len(blob))))
            blob.extend(np.ascontiguousarray(arr).tobytes())
            return name
        self.inits.append(_tensor_proto(name, arr, onnx_dtype, dims))
        return name

    def input(self, name, dtype, shape):
        self.inputs.append(_value_info(name, dtype, shape))
        return name

    def output(self, name, dtype, shape):
        self.outputs.append(_value_info(name, dtype, shape))

    def tobytes(self) -> bytes:
        g = b"".join(_f_bytes(1, n) for n in self.nodes) + _f_str(2, self.name) + b"".join(_f_bytes(5, t) for t in self.inits)
        g += b"".join(_f_bytes(11, i) for i in self.inputs) + b"".join(_f_bytes(12, o) for o in self.outputs)
        opsets = _f_bytes(8, _f_str(1, "") + _f_int(2, 21)) + _f_bytes(8, _f_str(1, "com.microsoft") + _f_int(2, 1))
        return _f_int(1, 10) + _f_str(2, "onyxia_b200") + opsets + _f_bytes(7, g)


def export_decoder(cfg, seed: int = 0) -> bytes:
    """The decoder of `models.build_decoder(cfg, seed)` as the ONNX graph an onnxruntime-genai style export of such
    a model has: contrib operators for the quantised projections and the attention, the sequence lengths derived
    from `attention_mask` by ReduceSum / Shape arithmetic. Same seeded weights, byte for byte."""
    from . import models
    w = OnnxWriter(cfg.name)
    adt, npa = cfg.act_dtype, cfg.np_act
    H, D, NH, KV = cfg.hidden, cfg.head_dim, cfg.heads, cfg.kv_heads
    B, S, P, T = "batch_size", "sequence_length", "past_sequence_length", "total_sequence_length"
    w.input("input_ids", ir.I64, [B, S])
    w.input("attention_mask", ir.I64, [B, T])
    for l in range(cfg.layers):
        w.input(f"past_key_values.{l}.key", adt, [B, KV, P, D])
        w.input(f"past_key_values.{l}.value", adt, [B, KV, P, D])

    def nbits(x, name, k, n, out):
        packed, scales, zp = models.nbits_arrays(cfg, seed, name, k, n)
        nb = (k + 31) // 32
        ins = [x, w.initializer(name + ".qweight", packed.reshape(n, nb, 16)), w.initializer(name + ".scales", scales)]
        if zp is not None:
            ins.append(w.initializer(name + ".qzeros", zp))
        return w.node("MatMulNBits", ins, [out], name=name, domain="com.microsoft", K=k, N=n, bits=4, block_size=32)

    def norm(x, name, out):
        return w.node("SimplifiedLayerNormalization", [x, w.initializer(name + ".weight", models.norm_array(cfg, seed, name, H))], [out],
                      name=name, epsilon=float(cfg.eps), axis=-1)

    w.initializer("axes_1", np.array([1], np.int64))
    w.initializer("one_i64", np.array([1], np.int64))
    w.initializer("idx_1", np.array(1, np.int64))
    w.node("ReduceSum", ["attention_mask", "axes_1"], ["mask_sum"], name="/model/attn_mask_reformat/seqlens", keepdims=0)
    w.node("Sub", ["mask_sum", "one_i64"], ["seqlens_i64"])
    w.node("Cast", ["seqlens_i64"], ["seqlens_k"], to=6)
    w.node("Shape", ["attention_mask"], ["mask_shape"])
    w.node("Gather", ["mask_shape", "idx_1"], ["total_i64"], axis=0)
    w.node("Cast", ["total_i64"], ["total_seq_len"], to=6)
    cos, sin = models.rope_caches(cfg)
    w.initializer("cos_cache", cos)
    w.initializer("sin_cache", sin)
    w.initializer("embed", models.embed_array(cfg, seed))
    x = w.node("Gather", ["embed", "input_ids"], ["x0"], name="/model/embed_tokens/Gather", axis=0)
    for l in range(cfg.layers):
        pre = f"/model/layers.{l}"
        h = norm(x, f"{pre}/input_layernorm", f"h{l}")
        q = nbits(h, f"{pre}/attn/q_proj", H, NH * D, f"q{l}")
        k = nbits(h, f"{pre}/attn/k_proj", H, KV * D, f"k{l}")
        v = nbits(h, f"{pre}/attn/v_proj", H, KV * D, f"v{l}")
        w.node("GroupQueryAttention", [q, k, v, f"past_key_values.{l}.key", f"past_key_values.{l}.value", "seqlens_k", "total_seq_len",
                                       "cos_cache", "sin_cache"], [f"attn{l}", f"present.{l}.key", f"present.{l}.value"],
               name=f"{pre}/attn/GroupQueryAttention", domain="com.microsoft", num_heads=NH, kv_num_heads=KV, scale=0.0,
               local_window_size=cfg.layer_window(l), do_rotary=1, rotary_interleaved=0)
        o = nbits(f"attn{l}", f"{pre}/attn/o_proj", NH * D, H, f"o{l}")
        if cfg.sandwich_norms:
            o = norm(o, f"{pre}/post_attention_layernorm", f"o_n{l}")
        x = w.node("Add", [x, o], [f"x_a{l}"], name=f"{pre}/residual_add_1")
        h2 = norm(x, f"{pre}/pre_feedforward_layernorm", f"h2_{l}")
        gate = nbits(h2, f"{pre}/mlp/gate_proj", H, cfg.ffn, f"gate{l}")
        up = nbits(h2, f"{pre}/mlp/up_proj", H, cfg.ffn, f"up{l}")
        act = w.node("Gelu", [gate], [f"act{l}"], name=f"{pre}/mlp/act_fn/Gelu", approximate="tanh" if cfg.gelu_tanh else "none")
        m = w.node("Mul", [act, up], [f"m{l}"], name=f"{pre}/mlp/Mul")
        down = nbits(m, f"{pre}/mlp/down_proj", cfg.ffn, H, f"down{l}")
        if cfg.sandwich_norms:
            down = norm(down, f"{pre}/post_feedforward_layernorm", f"down_n{l}")
        x = w.node("Add", [x, down], [f"x_b{l}"], name=f"{pre}/residual_add_2")
    x = norm(x, "/model/norm", "x_final")
    if cfg.last_logits_only:
        w.initializer("minus_1", np.array([-1], np.int64))
        w.initializer("int_max", np.array([(1 << 63) - 1], np.int64))
        x = w.node("Slice", [x, "minus_1", "int_max", "axes_1"], ["x_last"], name="/model/last_token/Slice")
    nbits(x, "/lm_head", H, cfg.vocab, "logits")
    w.output("logits", adt, [B, 1 if cfg.last_logits_only else S, cfg.vocab])
    for l in range(cfg.layers):
        w.output(f"present.{l}.key", adt, [B, KV, T, D])
        w.output(f"present.{l}.value", adt, [B, KV, T, D])
    return w.tobytes()
