// Data model, symbolic-dim algebra, graph surgery and binding.
// Reference behaviour: crates/onyxia-ir/src/{types,dim,prim,attrs,graph,fold}.rs
// and interp.rs:353-411 (bind_shapes).
#include "ir.hpp"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <sstream>

namespace ox {

// ───────────────────────────── errors ──────────────────────────────────
const char* err_prefix(ErrKind k) {
    switch (k) {
        case ErrKind::Ok: return "ok";
        case ErrKind::Shape: return "shape error";
        case ErrKind::InvalidGraph: return "invalid graph";
        case ErrKind::DType: return "dtype error";
        case ErrKind::Attribute: return "attribute error";
        case ErrKind::Binding: return "binding error";
        case ErrKind::Interp: return "interpreter error";
        case ErrKind::Unsupported: return "unsupported";
        case ErrKind::Runtime: return "runtime error";
    }
    return "error";
}

Error::Error(ErrKind k, const std::string& msg)
    : std::runtime_error(std::string(err_prefix(k)) + ": " + msg), kind(k), detail(msg) {}

// ───────────────────────────── dtypes ──────────────────────────────────
int dtype_bits(DType d) {
    switch (d) {
        case DType::F32: case DType::I32: case DType::U32: return 32;
        case DType::F16: return 16;
        case DType::I64: return 64;
        case DType::U8: case DType::I8: case DType::Bool: return 8;
        case DType::U4: case DType::I4: return 4;
    }
    return 0;
}

size_t dtype_storage_bytes(DType d, uint64_t n) {
    // 64-bit math regardless of pointer width (types.rs:73-76).
    return (size_t)((n * (uint64_t)dtype_bits(d) + 7) / 8);
}

const char* dtype_name(DType d) {
    static const char* names[] = {"f32", "f16", "i64", "i32", "u32", "u8", "i8", "bool", "u4", "i4"};
    return names[(int)d];
}

// ───────────────────────────── symbols ─────────────────────────────────
SymId SymbolTable::intern(const std::string& name) {
    auto it = by_name_.find(name);
    if (it != by_name_.end()) return it->second;
    SymId id = (SymId)names_.size();
    names_.push_back(name);
    by_name_[name] = id;
    return id;
}

SymId SymbolTable::fresh(const std::string& hint) {
    std::string name = hint + "$" + std::to_string(names_.size());
    while (by_name_.count(name)) name.push_back('\'');
    return intern(name);
}

std::optional<SymId> SymbolTable::get(const std::string& name) const {
    auto it = by_name_.find(name);
    if (it == by_name_.end()) return std::nullopt;
    return it->second;
}

void Bindings::bind(SymId s, uint64_t v) {
    for (auto& kv : items_) {
        if (kv.first == s) {
            if (kv.second != v)
                fail(ErrKind::Binding, "symbol bound to conflicting values " + std::to_string(kv.second) +
                                           " and " + std::to_string(v));
            return;
        }
    }
    items_.emplace_back(s, v);
}

std::optional<uint64_t> Bindings::get(SymId s) const {
    for (auto& kv : items_)
        if (kv.first == s) return kv.second;
    return std::nullopt;
}

// ───────────────────────────── DimExpr ─────────────────────────────────
DimExpr DimExpr::from_signed(int64_t c) {
    DimExpr e;
    if (c != 0) e.terms_.push_back(Term{{}, c});
    return e;
}

DimExpr DimExpr::sym(SymId s) {
    DimExpr e;
    e.terms_.push_back(Term{{s}, 1});
    return e;
}

std::optional<uint64_t> DimExpr::as_const() const {
    if (terms_.empty()) return 0;
    if (terms_.size() == 1 && terms_[0].syms.empty() && terms_[0].coeff >= 0) return (uint64_t)terms_[0].coeff;
    return std::nullopt;
}

bool DimExpr::is_const() const {
    for (auto& t : terms_)
        if (!t.syms.empty()) return false;
    return true;
}

std::optional<SymId> DimExpr::as_sym() const {
    if (terms_.size() == 1 && terms_[0].coeff == 1 && terms_[0].syms.size() == 1) return terms_[0].syms[0];
    return std::nullopt;
}

std::vector<SymId> DimExpr::syms() const {
    std::vector<SymId> out;
    for (auto& t : terms_) out.insert(out.end(), t.syms.begin(), t.syms.end());
    std::sort(out.begin(), out.end());
    out.erase(std::unique(out.begin(), out.end()), out.end());
    return out;
}

int64_t DimExpr::eval_signed(const Bindings& b) const {
    __int128 acc = 0;
    for (auto& t : terms_) {
        __int128 prod = t.coeff;
        for (SymId s : t.syms) {
            auto v = b.get(s);
            if (!v) fail(ErrKind::Binding, "unbound dimension symbol (id " + std::to_string(s) + ")");
            prod *= (__int128)*v;
        }
        acc += prod;
    }
    if (acc > (__int128)INT64_MAX || acc < (__int128)INT64_MIN)
        fail(ErrKind::Binding, "shape value overflows i64");
    return (int64_t)acc;
}

uint64_t DimExpr::eval(const Bindings& b) const {
    int64_t v = eval_signed(b);
    if (v < 0) fail(ErrKind::Binding, "dimension evaluated to negative value " + std::to_string(v));
    return (uint64_t)v;
}

bool DimExpr::try_eval(const Bindings& b, uint64_t* out, std::string* why) const {
    try {
        *out = eval(b);
        return true;
    } catch (const Error& e) {
        if (why) *why = e.what();
        return false;
    }
}

std::optional<DimExpr> DimExpr::div_exact(const DimExpr& divisor) const {
    if (divisor.terms_.size() != 1) return std::nullopt;  // not a monomial
    const Term& d = divisor.terms_[0];
    std::vector<Term> out;
    for (auto& t : terms_) {
        if (t.coeff % d.coeff != 0) return std::nullopt;
        std::vector<SymId> remaining = t.syms;
        for (SymId ds : d.syms) {
            auto pos = std::find(remaining.begin(), remaining.end(), ds);
            if (pos == remaining.end()) return std::nullopt;
            remaining.erase(pos);
        }
        out.push_back(Term{remaining, t.coeff / d.coeff});
    }
    return canonicalize(std::move(out));
}

DimExpr DimExpr::canonicalize(std::vector<Term> terms) {
    for (auto& t : terms) std::sort(t.syms.begin(), t.syms.end());
    // Higher symbol products first; any total order would do.
    std::stable_sort(terms.begin(), terms.end(), [](const Term& a, const Term& b) { return b.syms < a.syms; });
    DimExpr e;
    for (auto& t : terms) {
        if (!e.terms_.empty() && e.terms_.back().syms == t.syms)
            e.terms_.back().coeff += t.coeff;
        else
            e.terms_.push_back(std::move(t));
    }
    e.terms_.erase(std::remove_if(e.terms_.begin(), e.terms_.end(), [](const Term& t) { return t.coeff == 0; }),
                   e.terms_.end());
    return e;
}

DimExpr operator+(const DimExpr& a, const DimExpr& b) {
    std::vector<Term> t = a.terms_;
    t.insert(t.end(), b.terms_.begin(), b.terms_.end());
    return DimExpr::canonicalize(std::move(t));
}

DimExpr operator-(const DimExpr& a, const DimExpr& b) {
    std::vector<Term> t = a.terms_;
    for (auto x : b.terms_) {
        x.coeff = -x.coeff;
        t.push_back(std::move(x));
    }
    return DimExpr::canonicalize(std::move(t));
}

DimExpr operator*(const DimExpr& a, const DimExpr& b) {
    std::vector<Term> t;
    for (auto& x : a.terms_)
        for (auto& y : b.terms_) {
            Term z;
            z.syms = x.syms;
            z.syms.insert(z.syms.end(), y.syms.begin(), y.syms.end());
            z.coeff = x.coeff * y.coeff;
            t.push_back(std::move(z));
        }
    return DimExpr::canonicalize(std::move(t));
}

std::string DimExpr::to_string(const SymbolTable* table) const {
    if (terms_.empty()) return "0";
    std::ostringstream f;
    for (size_t i = 0; i < terms_.size(); i++) {
        const Term& t = terms_[i];
        if (i > 0)
            f << (t.coeff < 0 ? " - " : " + ");
        else if (t.coeff < 0)
            f << "-";
        uint64_t mag = t.coeff < 0 ? (uint64_t)(-(t.coeff + 1)) + 1 : (uint64_t)t.coeff;
        if (t.syms.empty()) {
            f << mag;
        } else {
            if (mag != 1) f << mag << "*";
            for (size_t j = 0; j < t.syms.size(); j++) {
                if (j > 0) f << "*";
                if (table)
                    f << table->name(t.syms[j]);
                else
                    f << "s" << t.syms[j];
            }
        }
    }
    return f.str();
}

SymShape fixed_shape(const std::vector<uint64_t>& dims) {
    SymShape s;
    for (auto d : dims) s.push_back(DimExpr::constant(d));
    return s;
}

DimExpr shape_numel(const SymShape& s) {
    DimExpr acc = DimExpr::constant(1);
    for (auto& d : s) acc = acc * d;
    return acc;
}

std::optional<std::vector<uint64_t>> shape_as_static(const SymShape& s) {
    std::vector<uint64_t> out;
    for (auto& d : s) {
        auto c = d.as_const();
        if (!c) return std::nullopt;
        out.push_back(*c);
    }
    return out;
}

std::vector<size_t> shape_eval(const SymShape& s, const Bindings& b) {
    std::vector<size_t> out;
    for (auto& d : s) out.push_back((size_t)d.eval(b));
    return out;
}

std::string shape_to_string(const SymShape& s, const SymbolTable* t) {
    std::string out = "[";
    for (size_t i = 0; i < s.size(); i++) {
        if (i) out += ", ";
        out += s[i].to_string(t);
    }
    return out + "]";
}

std::string TensorType::to_string(const SymbolTable* t) const {
    return std::string(dtype_name(dtype)) + shape_to_string(shape, t);
}

// ───────────────────────────── Prim ────────────────────────────────────
Prim Prim::unary(UnaryOp o) { Prim p; p.kind = PrimKind::Unary; p.op = (int)o; return p; }
Prim Prim::binary(BinaryOp o) { Prim p; p.kind = PrimKind::Binary; p.op = (int)o; return p; }
Prim Prim::compare(CmpOp o) { Prim p; p.kind = PrimKind::Compare; p.op = (int)o; return p; }
Prim Prim::select() { Prim p; p.kind = PrimKind::Select; return p; }
Prim Prim::cast(DType to) { Prim p; p.kind = PrimKind::Cast; p.dtype = to; return p; }
Prim Prim::matmul(bool ta, bool tb) { Prim p; p.kind = PrimKind::MatMul; p.trans_a = ta; p.trans_b = tb; return p; }
Prim Prim::reduce(ReduceOp o, std::vector<size_t> axes, bool keepdims) {
    Prim p; p.kind = PrimKind::Reduce; p.op = (int)o; p.axes = std::move(axes); p.keepdims = keepdims; return p;
}
Prim Prim::reshape(SymShape s) { Prim p; p.kind = PrimKind::Reshape; p.shape = std::move(s); return p; }
Prim Prim::transpose(std::vector<size_t> perm) { Prim p; p.kind = PrimKind::Transpose; p.axes = std::move(perm); return p; }
Prim Prim::broadcast(SymShape s) { Prim p; p.kind = PrimKind::Broadcast; p.shape = std::move(s); return p; }
Prim Prim::concat(size_t axis) { Prim p; p.kind = PrimKind::Concat; p.axis = axis; return p; }
Prim Prim::slice(std::vector<SliceSpec> specs) { Prim p; p.kind = PrimKind::Slice; p.specs = std::move(specs); return p; }
Prim Prim::gather(size_t axis) { Prim p; p.kind = PrimKind::Gather; p.axis = axis; return p; }
Prim Prim::scatter() { Prim p; p.kind = PrimKind::Scatter; return p; }
Prim Prim::iota(DimExpr len, DType dt) { Prim p; p.kind = PrimKind::Iota; p.len = std::move(len); p.dtype = dt; return p; }
Prim Prim::dim_values(SymShape exprs) { Prim p; p.kind = PrimKind::DimValues; p.shape = std::move(exprs); return p; }
Prim Prim::dequantize(size_t block_size, SymShape out_shape) {
    Prim p; p.kind = PrimKind::Dequantize; p.block_size = block_size; p.shape = std::move(out_shape); return p;
}

const char* Prim::name() const {
    static const char* un[] = {"neg", "abs", "sqrt", "rsqrt", "exp", "log", "sin", "cos", "tanh", "erf", "floor", "ceil", "not"};
    static const char* bi[] = {"add", "sub", "mul", "div", "pow", "max", "min", "and", "or", "xor"};
    static const char* cm[] = {"eq", "ne", "lt", "le", "gt", "ge"};
    static const char* rd[] = {"reduce_sum", "reduce_mean", "reduce_max", "reduce_min", "reduce_prod"};
    switch (kind) {
        case PrimKind::Unary: return un[op];
        case PrimKind::Binary: return bi[op];
        case PrimKind::Compare: return cm[op];
        case PrimKind::Select: return "select";
        case PrimKind::Cast: return "cast";
        case PrimKind::MatMul: return "matmul";
        case PrimKind::Reduce: return rd[op];
        case PrimKind::Reshape: return "reshape";
        case PrimKind::Transpose: return "transpose";
        case PrimKind::Broadcast: return "broadcast";
        case PrimKind::Concat: return "concat";
        case PrimKind::Slice: return "slice";
        case PrimKind::Gather: return "gather";
        case PrimKind::Scatter: return "scatter";
        case PrimKind::Iota: return "iota";
        case PrimKind::DimValues: return "dim_values";
        case PrimKind::Dequantize: return "dequantize";
    }
    return "?";
}

std::pair<size_t, size_t> Prim::arity() const {
    switch (kind) {
        case PrimKind::Unary: case PrimKind::Cast: case PrimKind::Reduce: case PrimKind::Reshape:
        case PrimKind::Transpose: case PrimKind::Broadcast: case PrimKind::Slice:
            return {1, 1};
        case PrimKind::Binary: case PrimKind::Compare: case PrimKind::MatMul: case PrimKind::Gather:
            return {2, 2};
        case PrimKind::Select: case PrimKind::Scatter:
            return {3, 3};
        case PrimKind::Iota: case PrimKind::DimValues:
            return {0, 0};
        case PrimKind::Dequantize:
            return {2, 3};
        case PrimKind::Concat:
            return {1, SIZE_MAX};
    }
    return {0, 0};
}

// ───────────────────────────── Attrs ───────────────────────────────────
static const char* attr_kind_name(AttrValue::Kind k) {
    static const char* n[] = {"int", "ints", "float", "floats", "str", "bool", "tensor"};
    return n[(int)k];
}
[[noreturn]] static void attr_missing(const std::string& name) {
    fail(ErrKind::Attribute, "missing attribute '" + name + "'");
}
[[noreturn]] static void attr_type(const std::string& name, const char* expected, const AttrValue& got) {
    fail(ErrKind::Attribute,
         "attribute '" + name + "': expected " + expected + ", found " + attr_kind_name(got.kind));
}

Attrs& Attrs::set(const std::string& name, AttrValue v) {
    for (auto& kv : items_)
        if (kv.first == name) {
            kv.second = std::move(v);
            return *this;
        }
    items_.emplace_back(name, std::move(v));
    return *this;
}
const AttrValue* Attrs::get(const std::string& name) const {
    for (auto& kv : items_)
        if (kv.first == name) return &kv.second;
    return nullptr;
}
int64_t Attrs::int_(const std::string& name) const {
    auto* v = get(name);
    if (!v) attr_missing(name);
    if (v->kind != AttrValue::Int) attr_type(name, "int", *v);
    return v->i;
}
int64_t Attrs::int_or(const std::string& name, int64_t dflt) const {
    auto* v = get(name);
    if (!v) return dflt;
    if (v->kind != AttrValue::Int) attr_type(name, "int", *v);
    return v->i;
}
double Attrs::float_(const std::string& name) const {
    auto* v = get(name);
    if (!v) attr_missing(name);
    if (v->kind != AttrValue::Float) attr_type(name, "float", *v);
    return v->f;
}
double Attrs::float_or(const std::string& name, double dflt) const {
    auto* v = get(name);
    if (!v) return dflt;
    if (v->kind != AttrValue::Float) attr_type(name, "float", *v);
    return v->f;
}
const std::string& Attrs::str(const std::string& name) const {
    auto* v = get(name);
    if (!v) attr_missing(name);
    if (v->kind != AttrValue::Str) attr_type(name, "str", *v);
    return v->s;
}
std::string Attrs::str_or(const std::string& name, const std::string& dflt) const {
    auto* v = get(name);
    if (!v || v->kind != AttrValue::Str) return dflt;  // decomp.rs:191 uses unwrap_or
    return v->s;
}
bool Attrs::bool_or(const std::string& name, bool dflt) const {
    auto* v = get(name);
    if (!v) return dflt;
    if (v->kind != AttrValue::Bool) attr_type(name, "bool", *v);
    return v->b;
}

// ───────────────────────────── ConstPool ───────────────────────────────
size_t ConstPool::expect_bytes(const TensorType& ty, const char* what) {
    auto dims = shape_as_static(ty.shape);
    if (!dims) fail(ErrKind::InvalidGraph, std::string(what) + " must have a static shape, got " + shape_to_string(ty.shape));
    uint64_t n = 1;
    for (auto d : *dims) n *= d;
    return dtype_storage_bytes(ty.dtype, n);
}

ConstId ConstPool::add(const TensorType& ty, std::vector<uint8_t> bytes) {
    size_t expect = expect_bytes(ty, "constant");
    if (bytes.size() != expect)
        fail(ErrKind::InvalidGraph, "constant data size mismatch: " + std::to_string(bytes.size()) + " bytes for " +
                                        ty.to_string() + " (expected " + std::to_string(expect) + ")");
    ConstEntry e;
    e.ty = ty;
    e.owned = std::make_shared<const std::vector<uint8_t>>(std::move(bytes));
    e.data = e.owned->data();
    e.nbytes = e.owned->size();
    entries_.push_back(std::move(e));
    return (ConstId)entries_.size() - 1;
}

ConstId ConstPool::add_borrowed(const TensorType& ty, const uint8_t* data, size_t nbytes) {
    size_t expect = expect_bytes(ty, "constant");
    if (nbytes != expect)
        fail(ErrKind::InvalidGraph, "constant data size mismatch: " + std::to_string(nbytes) + " bytes for " +
                                        ty.to_string() + " (expected " + std::to_string(expect) + ")");
    ConstEntry e;
    e.ty = ty;
    e.data = data;
    e.nbytes = nbytes;
    entries_.push_back(std::move(e));
    return (ConstId)entries_.size() - 1;
}

size_t ConstPool::total_bytes() const {
    size_t t = 0;
    for (auto& e : entries_) t += e.nbytes;
    return t;
}

void ConstPool::reinterpret(ConstId id, const TensorType& ty) {
    size_t expect = expect_bytes(ty, "reinterpret");
    if (entries_[id].nbytes != expect)
        fail(ErrKind::InvalidGraph, "reinterpret size mismatch: entry holds " + std::to_string(entries_[id].nbytes) +
                                        " bytes, " + ty.to_string() + " needs " + std::to_string(expect));
    entries_[id].ty = ty;
}

void ConstPool::release(ConstId id) {
    entries_[id].owned.reset();
    entries_[id].data = nullptr;
}

// ───────────────────────────── Module ──────────────────────────────────
std::vector<NodeId> Module::topo_order() const {
    enum State : uint8_t { Unvisited, Visiting, Done };
    std::vector<State> state(nodes.size(), Unvisited);
    std::vector<NodeId> order;
    order.reserve(nodes.size());
    std::vector<std::pair<NodeId, size_t>> stack;
    for (NodeId start = 0; start < nodes.size(); start++) {
        if (state[start] != Unvisited) continue;
        stack.clear();
        stack.emplace_back(start, 0);
        state[start] = Visiting;
        while (!stack.empty()) {
            NodeId node = stack.back().first;
            size_t next = stack.back().second;
            const auto& ins = nodes[node].inputs;
            if (next < ins.size()) {
                stack.back().second++;
                const Origin& o = values[ins[next]].origin;
                if (o.kind == Origin::Node) {
                    if (state[o.id] == Unvisited) {
                        state[o.id] = Visiting;
                        stack.emplace_back(o.id, 0);
                    } else if (state[o.id] == Visiting) {
                        fail(ErrKind::InvalidGraph, "graph contains a cycle");
                    }
                }
            } else {
                state[node] = Done;
                order.push_back(node);
                stack.pop_back();
            }
        }
    }
    return order;
}

void Module::replace_uses(ValueId old_v, ValueId new_v) {
    for (auto& n : nodes)
        for (auto& v : n.inputs)
            if (v == old_v) v = new_v;
    for (auto& o : outputs)
        if (o.second == old_v) o.second = new_v;
    if (!values[new_v].name) values[new_v].name = values[old_v].name;
}

void Module::remove_nodes(const std::unordered_set<NodeId>& dead) {
    const uint32_t NONE = UINT32_MAX;
    std::vector<uint32_t> node_remap(nodes.size(), NONE);
    std::vector<Node> kept_nodes;
    kept_nodes.reserve(nodes.size());
    for (size_t i = 0; i < nodes.size(); i++) {
        if (dead.count((NodeId)i)) continue;
        node_remap[i] = (uint32_t)kept_nodes.size();
        kept_nodes.push_back(std::move(nodes[i]));
    }
    std::vector<char> live(values.size(), 0);
    for (auto& io : inputs) live[io.second] = 1;
    for (auto& io : outputs) live[io.second] = 1;
    for (auto& n : kept_nodes) {
        for (auto v : n.inputs) live[v] = 1;
        for (auto v : n.outputs) live[v] = 1;
    }
    for (size_t i = 0; i < values.size(); i++)
        if (values[i].origin.kind == Origin::Node && node_remap[values[i].origin.id] == NONE) live[i] = 0;

    std::vector<uint32_t> value_remap(values.size(), NONE);
    std::vector<ValueDef> kept_values;
    for (size_t i = 0; i < values.size(); i++) {
        if (!live[i]) continue;
        value_remap[i] = (uint32_t)kept_values.size();
        kept_values.push_back(std::move(values[i]));
    }
    for (auto& d : kept_values)
        if (d.origin.kind == Origin::Node) d.origin.id = node_remap[d.origin.id];
    auto remap = [&](ValueId& v) {
        if (value_remap[v] == NONE) fail(ErrKind::InvalidGraph, "remove_nodes: surviving reference to a pruned value");
        v = value_remap[v];
    };
    for (auto& n : kept_nodes) {
        for (auto& v : n.inputs) remap(v);
        for (auto& v : n.outputs) remap(v);
    }
    for (auto& io : inputs) remap(io.second);
    for (auto& io : outputs) remap(io.second);
    nodes = std::move(kept_nodes);
    values = std::move(kept_values);
}

// A Transpose that swaps the last two axes of a MatMul operand (identity on the batch axes) becomes the
// MatMul's trans flag; the orphaned Transpose is left to eliminate_dead (crates/onyxia-ir/src/fold.rs:129-178).
// Tied-embedding exports feed the lm_head as MatMul(h, Transpose(W)): without the fold every run would
// materialise the transposed weight again.
bool fold_transpose_into_matmul(Module& m) {
    auto swaps_last_two = [](const std::vector<size_t>& perm) {
        const size_t r = perm.size();
        if (r < 2) return false;
        for (size_t i = 0; i + 2 < r; i++)
            if (perm[i] != i) return false;
        return perm[r - 2] == r - 1 && perm[r - 1] == r - 2;
    };
    bool changed = false;
    for (auto& n : m.nodes) {
        if (!n.is_prim || n.prim.kind != PrimKind::MatMul) continue;
        for (int side = 0; side < 2; side++) {
            const Origin& o = m.values[n.inputs[side]].origin;
            if (o.kind != Origin::Node) continue;
            const Node& prod = m.nodes[o.id];
            if (!prod.is_prim || prod.prim.kind != PrimKind::Transpose || !swaps_last_two(prod.prim.axes)) continue;
            n.inputs[side] = prod.inputs[0];
            if (side == 0) n.prim.trans_a = !n.prim.trans_a;
            else n.prim.trans_b = !n.prim.trans_b;
            changed = true;
        }
    }
    return changed;
}

size_t eliminate_dead(Module& m) {
    size_t removed = 0;
    for (;;) {
        std::vector<char> used(m.values.size(), 0);
        for (auto& o : m.outputs) used[o.second] = 1;
        for (auto& n : m.nodes)
            for (auto v : n.inputs) used[v] = 1;
        std::unordered_set<NodeId> dead;
        for (NodeId i = 0; i < m.nodes.size(); i++) {
            bool any = false;
            for (auto v : m.nodes[i].outputs) any |= (bool)used[v];
            if (!any) dead.insert(i);
        }
        if (dead.empty()) return removed;
        removed += dead.size();
        m.remove_nodes(dead);
    }
}

// ───────────────────────────── binding ─────────────────────────────────
static std::string shape_dbg(const size_t* s, size_t r) {
    std::string out = "[";
    for (size_t i = 0; i < r; i++) {
        if (i) out += ", ";
        out += std::to_string(s[i]);
    }
    return out + "]";
}

Bindings bind_shapes(const Module& m, const std::vector<InputDesc>& inputs) {
    Bindings b;
    for (int verify_only = 0; verify_only < 2; verify_only++) {
        for (auto& in : m.inputs) {
            const std::string& name = in.first;
            const InputDesc* got = nullptr;
            for (auto& d : inputs)
                if (name == d.name) {
                    got = &d;
                    break;
                }
            if (!got) fail(ErrKind::Binding, "missing input '" + name + "'");
            const TensorType& declared = m.values[in.second].ty;
            if (declared.dtype != got->dtype)
                fail(ErrKind::Binding, "input '" + name + "': dtype " + dtype_name(declared.dtype) + " declared, " +
                                           dtype_name(got->dtype) + " provided");
            if (declared.shape.size() != got->rank)
                fail(ErrKind::Binding, "input '" + name + "': rank " + std::to_string(declared.shape.size()) +
                                           " declared, shape " + shape_dbg(got->shape, got->rank) + " provided");
            for (size_t i = 0; i < got->rank; i++) {
                const DimExpr& expr = declared.shape[i];
                size_t concrete = got->shape[i];
                if (auto s = expr.as_sym()) {
                    if (!verify_only) {
                        try {
                            b.bind(*s, concrete);
                        } catch (const Error& e) {
                            fail(ErrKind::Binding, "input '" + name + "': " + e.what());
                        }
                    }
                } else if (verify_only) {
                    uint64_t expect = 0;
                    std::string why;
                    if (!expr.try_eval(b, &expect, &why))
                        fail(ErrKind::Binding, "input '" + name + "': cannot resolve declared dim " +
                                                   expr.to_string(&m.symbols) + ": " + why);
                    if (expect != concrete)
                        fail(ErrKind::Binding, "input '" + name + "': dim " + expr.to_string(&m.symbols) + " = " +
                                                   std::to_string(expect) + " but got " + std::to_string(concrete));
                }
            }
        }
    }
    for (auto& c : m.constraints) {
        int64_t l, r;
        try {
            l = c.left.eval_signed(b);
        } catch (const Error& e) {
            fail(ErrKind::Binding, c.context + ": cannot resolve " + c.left.to_string(&m.symbols) + ": " + e.what());
        }
        try {
            r = c.right.eval_signed(b);
        } catch (const Error& e) {
            fail(ErrKind::Binding, c.context + ": cannot resolve " + c.right.to_string(&m.symbols) + ": " + e.what());
        }
        if (l != r)
            fail(ErrKind::Binding, c.context + ": " + c.left.to_string(&m.symbols) + " = " + std::to_string(l) +
                                       " but " + c.right.to_string(&m.symbols) + " = " + std::to_string(r));
    }
    return b;
}

// ───────────────────────────── builder ─────────────────────────────────
Module GraphBuilder::finish() {
    validate(module_);
    return std::move(module_);
}

void GraphBuilder::constrain(const DimExpr& l, const DimExpr& r, const std::string& ctx) {
    if (l == r) return;  // holds structurally
    module_.constraints.push_back(DimConstraint{l, r, ctx});
}

ValueId GraphBuilder::input(const std::string& name, const TensorType& ty) {
    ValueDef d;
    d.name = name;
    d.ty = ty;
    d.origin.kind = Origin::Input;
    ValueId id = module_.add_value(std::move(d));
    module_.inputs.emplace_back(name, id);
    return id;
}

ValueId GraphBuilder::constant(const TensorType& ty, std::vector<uint8_t> bytes) {
    ConstId cid = module_.consts.add(ty, std::move(bytes));
    ValueDef d;
    d.ty = ty;
    d.origin.kind = Origin::Const;
    d.origin.id = cid;
    return module_.add_value(std::move(d));
}

ValueId GraphBuilder::constant_borrowed(const TensorType& ty, const uint8_t* data, size_t nbytes) {
    ConstId cid = module_.consts.add_borrowed(ty, data, nbytes);
    ValueDef d;
    d.ty = ty;
    d.origin.kind = Origin::Const;
    d.origin.id = cid;
    return module_.add_value(std::move(d));
}

ValueId GraphBuilder::prim(const Prim& p, const std::vector<ValueId>& inputs) {
    std::vector<const TensorType*> tys;
    for (auto v : inputs) {
        if (v >= module_.values.size()) fail(ErrKind::InvalidGraph, "input value id out of range");
        tys.push_back(&module_.values[v].ty);
    }
    std::vector<TensorType> outs;
    try {
        outs = infer_prim(p, tys);
    } catch (const Error& e) {
        fail(ErrKind::Shape, std::string(e.what()) + " (while building '" + p.name() + "' node" +
                                 (loc_name_ ? " for " + *loc_name_ : std::string()) + ")");
    }
    NodeId nid = (NodeId)module_.nodes.size();
    Node n;
    n.is_prim = true;
    n.prim = p;
    n.inputs = inputs;
    n.loc_name = loc_name_;
    n.loc_op = loc_op_;
    for (size_t i = 0; i < outs.size(); i++) {
        ValueDef d;
        d.ty = outs[i];
        d.origin.kind = Origin::Node;
        d.origin.id = nid;
        d.origin.output = (uint32_t)i;
        n.outputs.push_back(module_.add_value(std::move(d)));
    }
    ValueId out = n.outputs[0];
    module_.add_node(std::move(n));
    return out;
}

std::vector<ValueId> GraphBuilder::composite(const std::string& name, const Attrs& attrs,
                                             const std::vector<ValueId>& inputs,
                                             const std::vector<TensorType>& out_tys) {
    if (out_tys.empty()) fail(ErrKind::InvalidGraph, "composite '" + name + "' must declare at least one output");
    for (auto v : inputs)
        if (v >= module_.values.size()) fail(ErrKind::InvalidGraph, "input value id out of range");
    NodeId nid = (NodeId)module_.nodes.size();
    Node n;
    n.is_prim = false;
    n.composite.name = name;
    n.composite.attrs = attrs;
    n.inputs = inputs;
    n.loc_name = loc_name_;
    n.loc_op = loc_op_;
    for (size_t i = 0; i < out_tys.size(); i++) {
        ValueDef d;
        d.ty = out_tys[i];
        d.origin.kind = Origin::Node;
        d.origin.id = nid;
        d.origin.output = (uint32_t)i;
        n.outputs.push_back(module_.add_value(std::move(d)));
    }
    std::vector<ValueId> outs = n.outputs;
    module_.add_node(std::move(n));
    return outs;
}

void GraphBuilder::output(const std::string& name, ValueId v) {
    if (v >= module_.values.size()) fail(ErrKind::InvalidGraph, "output value id out of range");
    if (!module_.values[v].name) module_.values[v].name = name;
    module_.outputs.emplace_back(name, v);
}

// ───────────────────────────── half floats ─────────────────────────────
uint16_t f64_to_f16_bits(double v) {
    uint64_t x;
    std::memcpy(&x, &v, 8);
    uint16_t sign = (uint16_t)((x >> 48) & 0x8000);
    uint64_t mant = x & 0x000FFFFFFFFFFFFFull;
    int exp = (int)((x >> 52) & 0x7FF);
    if (exp == 0x7FF) {  // inf / nan
        if (mant == 0) return sign | 0x7C00;
        uint16_t m = (uint16_t)(mant >> 42);
        return sign | 0x7C00 | 0x0200 | m;  // quiet NaN
    }
    int e = exp - 1023;  // unbiased
    if (e > 15) return sign | 0x7C00;  // overflow → inf
    if (e >= -14) {
        // normal half: keep 10 mantissa bits, round to nearest even on the 42 dropped bits
        uint64_t m = mant >> 42;
        uint64_t rest = mant & ((1ull << 42) - 1);
        uint64_t halfway = 1ull << 41;
        uint32_t h = ((uint32_t)(e + 15) << 10) | (uint32_t)m;
        if (rest > halfway || (rest == halfway && (h & 1))) h++;  // may carry into exponent / inf: correct
        return sign | (uint16_t)h;
    }
    if (e < -25) return sign;  // below half of the smallest subnormal → ±0
    // subnormal half: value = full_mant * 2^(e-52), target unit 2^-24
    uint64_t full = mant | (1ull << 52);
    int shift = (-14 - e) + 42;  // bits dropped
    uint64_t m = full >> shift;
    uint64_t rest = full & ((1ull << shift) - 1);
    uint64_t halfway = 1ull << (shift - 1);
    uint32_t h = (uint32_t)m;
    if (rest > halfway || (rest == halfway && (h & 1))) h++;
    return sign | (uint16_t)h;
}

double f16_bits_to_f64(uint16_t h) {
    int sign = (h >> 15) & 1;
    int exp = (h >> 10) & 0x1F;
    int mant = h & 0x3FF;
    double v;
    if (exp == 0)
        v = std::ldexp((double)mant, -24);
    else if (exp == 31)
        v = mant ? std::nan("") : INFINITY;
    else
        v = std::ldexp((double)(mant | 0x400), exp - 25);
    return sign ? -v : v;
}

}  // namespace ox
