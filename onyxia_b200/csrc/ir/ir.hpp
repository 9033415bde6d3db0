// Host-side data model of the Onyxia IR, as it crosses the backend boundary.
//
// Mirrors the reference crate `onyxia-ir`:
//   dtypes            crates/onyxia-ir/src/types.rs:13-76
//   symbolic dims     crates/onyxia-ir/src/dim.rs:131-308
//   primitives        crates/onyxia-ir/src/prim.rs:130-296
//   attributes        crates/onyxia-ir/src/attrs.rs:12-166
//   module / values   crates/onyxia-ir/src/graph.rs:60-475
//   errors            crates/onyxia-ir/src/lib.rs:55-89
//
// Everything here is plain C++17 with no device dependency; the CUDA backend
// and the CPU oracle both build on it.
#pragma once
#include <cstddef>
#include <cstdint>
#include <functional>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <utility>
#include <vector>

namespace ox {

// ───────────────────────────── errors ──────────────────────────────────
enum class ErrKind : int {
    Ok = 0,
    Shape = 1,
    InvalidGraph = 2,
    DType = 3,
    Attribute = 4,
    Binding = 5,
    Interp = 6,
    Unsupported = 7,
    Runtime = 8,
};

const char* err_prefix(ErrKind k);

struct Error : std::runtime_error {
    ErrKind kind;
    std::string detail;  // message without the kind prefix
    Error(ErrKind k, const std::string& msg);
};

[[noreturn]] inline void fail(ErrKind k, const std::string& msg) { throw Error(k, msg); }

// ───────────────────────────── dtypes ──────────────────────────────────
enum class DType : int { F32 = 0, F16, I64, I32, U32, U8, I8, Bool, U4, I4 };
constexpr int kNumDTypes = 10;

int dtype_bits(DType d);
inline bool dtype_is_float(DType d) { return d == DType::F32 || d == DType::F16; }
inline bool dtype_is_int(DType d) {
    return d == DType::I64 || d == DType::I32 || d == DType::U32 || d == DType::U8 ||
           d == DType::I8 || d == DType::U4 || d == DType::I4;
}
inline bool dtype_is_packed(DType d) { return d == DType::U4 || d == DType::I4; }
// Storage bytes for n logical elements; packed types round the total up.
size_t dtype_storage_bytes(DType d, uint64_t n);
const char* dtype_name(DType d);

// ───────────────────────── symbolic dimensions ─────────────────────────
using SymId = uint32_t;

class SymbolTable {
public:
    SymId intern(const std::string& name);
    SymId fresh(const std::string& hint);
    const std::string& name(SymId id) const { return names_[id]; }
    std::optional<SymId> get(const std::string& name) const;
    size_t size() const { return names_.size(); }
    const std::vector<std::string>& names() const { return names_; }

private:
    std::vector<std::string> names_;
    std::unordered_map<std::string, SymId> by_name_;
};

// Concrete symbol values for one run.
class Bindings {
public:
    // Throws Binding on a conflicting re-bind.
    void bind(SymId s, uint64_t v);
    std::optional<uint64_t> get(SymId s) const;
    const std::vector<std::pair<SymId, uint64_t>>& items() const { return items_; }

private:
    std::vector<std::pair<SymId, uint64_t>> items_;  // tiny; linear scan
};

struct Term {
    std::vector<SymId> syms;  // sorted, with multiplicity
    int64_t coeff = 0;        // never 0 in canonical form
    bool operator==(const Term& o) const { return coeff == o.coeff && syms == o.syms; }
};

// Integer polynomial over symbols in canonical form: structural equality is
// semantic equality.
class DimExpr {
public:
    DimExpr() = default;  // the constant 0
    static DimExpr constant(uint64_t c) { return from_signed((int64_t)c); }
    static DimExpr from_signed(int64_t c);
    static DimExpr sym(SymId s);
    static DimExpr from_terms(std::vector<Term> terms) { return canonicalize(std::move(terms)); }

    std::optional<uint64_t> as_const() const;
    bool is_const() const;
    std::optional<SymId> as_sym() const;
    std::vector<SymId> syms() const;
    uint64_t eval(const Bindings& b) const;       // throws Binding if unbound or negative
    int64_t eval_signed(const Bindings& b) const;  // throws Binding if unbound
    bool try_eval(const Bindings& b, uint64_t* out, std::string* why) const;
    std::optional<DimExpr> div_exact(const DimExpr& divisor) const;
    std::string to_string(const SymbolTable* table = nullptr) const;
    const std::vector<Term>& terms() const { return terms_; }

    bool operator==(const DimExpr& o) const { return terms_ == o.terms_; }
    bool operator!=(const DimExpr& o) const { return !(*this == o); }
    friend DimExpr operator+(const DimExpr& a, const DimExpr& b);
    friend DimExpr operator-(const DimExpr& a, const DimExpr& b);
    friend DimExpr operator*(const DimExpr& a, const DimExpr& b);

private:
    static DimExpr canonicalize(std::vector<Term> terms);
    std::vector<Term> terms_;
};

using SymShape = std::vector<DimExpr>;
SymShape fixed_shape(const std::vector<uint64_t>& dims);
DimExpr shape_numel(const SymShape& s);
std::optional<std::vector<uint64_t>> shape_as_static(const SymShape& s);
std::vector<size_t> shape_eval(const SymShape& s, const Bindings& b);
std::string shape_to_string(const SymShape& s, const SymbolTable* t = nullptr);

struct TensorType {
    DType dtype = DType::F32;
    SymShape shape;
    bool operator==(const TensorType& o) const { return dtype == o.dtype && shape == o.shape; }
    bool operator!=(const TensorType& o) const { return !(*this == o); }
    std::string to_string(const SymbolTable* t = nullptr) const;
};

// ───────────────────────────── primitives ──────────────────────────────
enum class UnaryOp : int { Neg, Abs, Sqrt, Rsqrt, Exp, Log, Sin, Cos, Tanh, Erf, Floor, Ceil, Not };
enum class BinaryOp : int { Add, Sub, Mul, Div, Pow, Max, Min, And, Or, Xor };
enum class CmpOp : int { Eq, Ne, Lt, Le, Gt, Ge };
enum class ReduceOp : int { Sum, Mean, Max, Min, Prod };

enum class PrimKind : int {
    Unary, Binary, Compare, Select, Cast, MatMul, Reduce, Reshape, Transpose, Broadcast,
    Concat, Slice, Gather, Scatter, Iota, DimValues, Dequantize,
};
constexpr int kNumPrimKinds = 17;

struct SliceSpec {
    size_t axis = 0;
    DimExpr start, end;
    int64_t step = 1;
};

// One tagged struct instead of a sum type: only the fields of `kind` matter.
struct Prim {
    PrimKind kind = PrimKind::Unary;
    int op = 0;                    // UnaryOp / BinaryOp / CmpOp / ReduceOp
    DType dtype = DType::F32;      // Cast.to, Iota.dtype
    bool trans_a = false, trans_b = false;  // MatMul
    std::vector<size_t> axes;      // Reduce.axes, Transpose.perm
    bool keepdims = false;         // Reduce
    SymShape shape;                // Reshape / Broadcast target, Dequantize.out_shape, DimValues.exprs
    size_t axis = 0;               // Concat / Gather
    std::vector<SliceSpec> specs;  // Slice
    DimExpr len;                   // Iota
    size_t block_size = 0;         // Dequantize

    static Prim unary(UnaryOp o);
    static Prim binary(BinaryOp o);
    static Prim compare(CmpOp o);
    static Prim select();
    static Prim cast(DType to);
    static Prim matmul(bool ta, bool tb);
    static Prim reduce(ReduceOp o, std::vector<size_t> axes, bool keepdims);
    static Prim reshape(SymShape s);
    static Prim transpose(std::vector<size_t> perm);
    static Prim broadcast(SymShape s);
    static Prim concat(size_t axis);
    static Prim slice(std::vector<SliceSpec> specs);
    static Prim gather(size_t axis);
    static Prim scatter();
    static Prim iota(DimExpr len, DType dt);
    static Prim dim_values(SymShape exprs);
    static Prim dequantize(size_t block_size, SymShape out_shape);

    const char* name() const;
    // (min, max) inputs; max == SIZE_MAX for Concat.
    std::pair<size_t, size_t> arity() const;
};

// ───────────────────────────── attributes ──────────────────────────────
struct AttrValue {
    enum Kind { Int, Ints, Float, Floats, Str, Bool, Tensor } kind = Int;
    int64_t i = 0;
    double f = 0;
    bool b = false;
    std::string s;
    std::vector<int64_t> ints;
    std::vector<double> floats;
    static AttrValue of_int(int64_t v) { AttrValue a; a.kind = Int; a.i = v; return a; }
    static AttrValue of_float(double v) { AttrValue a; a.kind = Float; a.f = v; return a; }
    static AttrValue of_str(std::string v) { AttrValue a; a.kind = Str; a.s = std::move(v); return a; }
    static AttrValue of_bool(bool v) { AttrValue a; a.kind = Bool; a.b = v; return a; }
    static AttrValue of_ints(std::vector<int64_t> v) { AttrValue a; a.kind = Ints; a.ints = std::move(v); return a; }
    static AttrValue of_floats(std::vector<double> v) { AttrValue a; a.kind = Floats; a.floats = std::move(v); return a; }
    static AttrValue of_tensor(int64_t const_id) { AttrValue a; a.kind = Tensor; a.i = const_id; return a; }
};

// Ordered name → value map; lookups are linear (attribute counts are tiny).
class Attrs {
public:
    Attrs& set(const std::string& name, AttrValue v);
    const AttrValue* get(const std::string& name) const;
    int64_t int_(const std::string& name) const;
    int64_t int_or(const std::string& name, int64_t dflt) const;
    double float_(const std::string& name) const;
    double float_or(const std::string& name, double dflt) const;
    const std::string& str(const std::string& name) const;
    std::string str_or(const std::string& name, const std::string& dflt) const;
    bool bool_or(const std::string& name, bool dflt) const;
    const std::vector<std::pair<std::string, AttrValue>>& items() const { return items_; }

private:
    std::vector<std::pair<std::string, AttrValue>> items_;
};

// ─────────────────────────────── graph ─────────────────────────────────
using ValueId = uint32_t;
using NodeId = uint32_t;
using ConstId = uint32_t;

struct Origin {
    enum Kind { Input, Const, Node } kind = Input;
    uint32_t id = 0;      // ConstId or NodeId
    uint32_t output = 0;  // output slot for Node
    bool operator==(const Origin& o) const {
        return kind == o.kind && (kind == Input || (id == o.id && (kind == Const || output == o.output)));
    }
};

struct ValueDef {
    std::optional<std::string> name;
    TensorType ty;
    Origin origin;
};

struct Composite {
    std::string name;
    Attrs attrs;
};

struct Node {
    bool is_prim = true;
    Prim prim;
    Composite composite;
    std::vector<ValueId> inputs;
    std::vector<ValueId> outputs;
    std::optional<std::string> loc_name;   // original node name
    std::optional<std::string> loc_op;     // original op type
};

// Constant bytes are shared, immutable and possibly borrowed from the caller
// (a borrowed entry must outlive every module copy that references it).
struct ConstEntry {
    TensorType ty;
    std::shared_ptr<const std::vector<uint8_t>> owned;
    const uint8_t* data = nullptr;
    size_t nbytes = 0;
};

class ConstPool {
public:
    ConstId add(const TensorType& ty, std::vector<uint8_t> bytes);
    ConstId add_borrowed(const TensorType& ty, const uint8_t* data, size_t nbytes);
    const TensorType& ty(ConstId id) const { return entries_[id].ty; }
    const uint8_t* bytes(ConstId id) const { return entries_[id].data; }
    size_t nbytes(ConstId id) const { return entries_[id].nbytes; }
    size_t size() const { return entries_.size(); }
    size_t total_bytes() const;
    void reinterpret(ConstId id, const TensorType& ty);
    // Drop the host bytes of one entry (after the backend uploaded it).
    void release(ConstId id);

private:
    static size_t expect_bytes(const TensorType& ty, const char* what);
    std::vector<ConstEntry> entries_;
};

struct DimConstraint {
    DimExpr left, right;
    std::string context;
};

struct Module {
    std::vector<ValueDef> values;
    std::vector<Node> nodes;
    ConstPool consts;
    SymbolTable symbols;
    std::vector<std::pair<std::string, ValueId>> inputs;
    std::vector<std::pair<std::string, ValueId>> outputs;
    std::vector<DimConstraint> constraints;

    ValueId add_value(ValueDef d) { values.push_back(std::move(d)); return (ValueId)values.size() - 1; }
    NodeId add_node(Node n) { nodes.push_back(std::move(n)); return (NodeId)nodes.size() - 1; }
    std::vector<NodeId> topo_order() const;  // throws InvalidGraph on a cycle
    void replace_uses(ValueId old_v, ValueId new_v);
    void remove_nodes(const std::unordered_set<NodeId>& dead);
};

// The part of `m` that rank `rank` of `tp` tensor-parallel ranks executes:
// MatMulNBits pairs split along N then K with an `onyxia.AllReduce` composite
// after every K-split node, attention on the rank's heads and its share of the
// KV cache, everything else replicated (see tp.cpp).
Module tp_partition(const Module& m, int tp, int rank);
void tp_partition_stats(const Module& m, int tp, size_t* col, size_t* row, size_t* attn);

// Remove nodes none of whose outputs are consumed; returns how many.
size_t eliminate_dead(Module& m);
bool fold_transpose_into_matmul(Module& m);

// ───────────────────────── inference / validation ──────────────────────
// Total over the primitive set (crates/onyxia-ir/src/infer.rs:26-318).
std::vector<TensorType> infer_prim(const Prim& p, const std::vector<const TensorType*>& inputs);
SymShape broadcast_shapes(const SymShape& a, const SymShape& b);
// Structural validation (crates/onyxia-ir/src/validate.rs:15-140).
void validate(const Module& m);

// Unify declared input shapes with concrete ones
// (crates/onyxia-ir/src/interp.rs:353-411).
struct InputDesc {
    const char* name;
    DType dtype;
    const size_t* shape;
    size_t rank;
};
Bindings bind_shapes(const Module& m, const std::vector<InputDesc>& inputs);

// ───────────────────────────── builder ─────────────────────────────────
// Eagerly typed construction (crates/onyxia-ir/src/builder.rs:39-360).
class GraphBuilder {
public:
    GraphBuilder() = default;
    explicit GraphBuilder(Module m) : module_(std::move(m)) {}
    Module into_module() { return std::move(module_); }
    Module finish();
    Module& module() { return module_; }
    const TensorType& ty(ValueId v) const { return module_.values[v].ty; }
    DimExpr sym(const std::string& name) { return DimExpr::sym(module_.symbols.intern(name)); }
    void set_loc(std::optional<std::string> name, std::optional<std::string> op) {
        loc_name_ = std::move(name); loc_op_ = std::move(op);
    }
    void constrain(const DimExpr& l, const DimExpr& r, const std::string& ctx);
    ValueId input(const std::string& name, const TensorType& ty);
    ValueId constant(const TensorType& ty, std::vector<uint8_t> bytes);
    ValueId constant_borrowed(const TensorType& ty, const uint8_t* data, size_t nbytes);
    ValueId prim(const Prim& p, const std::vector<ValueId>& inputs);
    std::vector<ValueId> composite(const std::string& name, const Attrs& attrs,
                                   const std::vector<ValueId>& inputs,
                                   const std::vector<TensorType>& out_tys);
    void output(const std::string& name, ValueId v);

    // sugar
    ValueId unary(UnaryOp o, ValueId x) { return prim(Prim::unary(o), {x}); }
    ValueId binary(BinaryOp o, ValueId a, ValueId b) { return prim(Prim::binary(o), {a, b}); }
    ValueId add(ValueId a, ValueId b) { return binary(BinaryOp::Add, a, b); }
    ValueId sub(ValueId a, ValueId b) { return binary(BinaryOp::Sub, a, b); }
    ValueId mul(ValueId a, ValueId b) { return binary(BinaryOp::Mul, a, b); }
    ValueId div(ValueId a, ValueId b) { return binary(BinaryOp::Div, a, b); }
    ValueId cmp(CmpOp o, ValueId a, ValueId b) { return prim(Prim::compare(o), {a, b}); }
    ValueId select(ValueId c, ValueId a, ValueId b) { return prim(Prim::select(), {c, a, b}); }
    ValueId cast(ValueId x, DType to) { return prim(Prim::cast(to), {x}); }
    ValueId matmul(ValueId a, ValueId b, bool ta = false, bool tb = false) {
        return prim(Prim::matmul(ta, tb), {a, b});
    }
    ValueId reduce(ReduceOp o, ValueId x, std::vector<size_t> axes, bool keep) {
        return prim(Prim::reduce(o, std::move(axes), keep), {x});
    }
    ValueId reshape(ValueId x, SymShape s) { return prim(Prim::reshape(std::move(s)), {x}); }
    ValueId transpose(ValueId x, std::vector<size_t> perm) { return prim(Prim::transpose(std::move(perm)), {x}); }
    ValueId broadcast(ValueId x, SymShape s) { return prim(Prim::broadcast(std::move(s)), {x}); }
    ValueId concat(const std::vector<ValueId>& xs, size_t axis) { return prim(Prim::concat(axis), xs); }
    ValueId slice(ValueId x, std::vector<SliceSpec> specs) { return prim(Prim::slice(std::move(specs)), {x}); }
    ValueId gather(ValueId data, ValueId idx, size_t axis) { return prim(Prim::gather(axis), {data, idx}); }
    ValueId iota(DimExpr len, DType dt) { return prim(Prim::iota(std::move(len), dt), {}); }

private:
    Module module_;
    std::optional<std::string> loc_name_, loc_op_;
};

// ─────────────────────────── decompositions ────────────────────────────
// crates/onyxia-ir/src/decomp.rs:24-133
using DecompFn = std::function<std::vector<ValueId>(const Composite&, const std::vector<ValueId>&, GraphBuilder&)>;

class DecompositionRegistry {
public:
    void register_(const std::string& name, DecompFn f) { map_[name] = std::move(f); }
    const DecompFn* get(const std::string& name) const;

private:
    std::unordered_map<std::string, DecompFn> map_;
};

const DecompositionRegistry& standard_decompositions();

// Inline composites until every remaining composite node satisfies `supports`.
// The predicate sees the whole node so a backend can keep a composite only for
// the operand types its kernel handles.
Module inline_composites(Module m, const DecompositionRegistry& reg,
                         const std::function<bool(const Module&, const Node&)>& supports);

// ───────────────────────────── half floats ─────────────────────────────
// IEEE binary16 <-> double, round-to-nearest-even directly from f64 (no
// intermediate f32 rounding), overflow to ±inf, subnormals kept. Stands in for
// `half::f16::from_f64` / `to_f64` (half 2.7.1), used by the reference at
// crates/onyxia-ir/src/interp.rs:153,230 and decomp.rs:141.
uint16_t f64_to_f16_bits(double v);
double f16_bits_to_f64(uint16_t h);

}  // namespace ox
