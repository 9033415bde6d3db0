// extern "C" module-construction calls of onyxia_cuda.h, over the C++ IR.
#include "module_api.hpp"

#include <cstring>

using namespace ox;

namespace ox {

thread_local std::string g_last_error;

int set_error(const Error& e) {
    g_last_error = e.what();
    return (int)e.kind;
}
int set_error(ErrKind k, const std::string& msg) {
    g_last_error = std::string(err_prefix(k)) + ": " + msg;
    return (int)k;
}

DimExpr dim_from_c(const ox_dimexpr& e) {
    std::vector<Term> terms;
    for (int i = 0; i < e.n_terms; i++) {
        const ox_dimterm& t = e.terms[i];
        if (t.n_syms < 0 || t.n_syms > OX_MAX_TERM_SYMS) fail(ErrKind::Shape, "dim term has too many symbols");
        Term x;
        x.coeff = t.coeff;
        for (int j = 0; j < t.n_syms; j++) x.syms.push_back((SymId)t.syms[j]);
        terms.push_back(std::move(x));
    }
    return DimExpr::from_terms(std::move(terms));
}

static SymShape shape_from_c(const ox_dimexpr* dims, int rank) {
    SymShape s;
    for (int i = 0; i < rank; i++) s.push_back(dim_from_c(dims[i]));
    return s;
}

static DType dtype_from_c(int32_t d) {
    if (d < 0 || d >= kNumDTypes) fail(ErrKind::DType, "unknown dtype code " + std::to_string(d));
    return (DType)d;
}

Prim prim_from_c(const ox_prim_desc& d) {
    if (d.kind < 0 || d.kind >= kNumPrimKinds) fail(ErrKind::InvalidGraph, "unknown primitive kind");
    Prim p;
    p.kind = (PrimKind)d.kind;
    p.op = d.op;
    auto check_op = [&](int n) {
        if (d.op < 0 || d.op >= n) fail(ErrKind::InvalidGraph, "operator code out of range");
    };
    switch (p.kind) {
        case PrimKind::Unary: check_op(13); break;
        case PrimKind::Binary: check_op(10); break;
        case PrimKind::Compare: check_op(6); break;
        case PrimKind::Reduce: check_op(5); break;
        default: break;
    }
    p.dtype = dtype_from_c(d.dtype);
    p.trans_a = d.trans_a != 0;
    p.trans_b = d.trans_b != 0;
    p.keepdims = d.keepdims != 0;
    for (int i = 0; i < d.n_axes; i++) p.axes.push_back((size_t)d.axes[i]);
    p.shape = shape_from_c(d.shape, d.n_shape);
    p.axis = (size_t)d.axis;
    for (int i = 0; i < d.n_specs; i++) {
        SliceSpec s;
        s.axis = (size_t)d.specs[i].axis;
        s.start = dim_from_c(d.specs[i].start);
        s.end = dim_from_c(d.specs[i].end);
        s.step = d.specs[i].step;
        p.specs.push_back(std::move(s));
    }
    p.len = dim_from_c(d.len);
    p.block_size = (size_t)d.block_size;
    return p;
}

}  // namespace ox

#define OX_TRY try {
#define OX_CATCH                                                        \
    }                                                                   \
    catch (const ox::Error& e) { return (ox_status)ox::set_error(e); }  \
    catch (const std::exception& e) {                                   \
        return (ox_status)ox::set_error(ErrKind::Runtime, e.what());    \
    }

extern "C" {

const char* ox_last_error(void) { return g_last_error.c_str(); }

ox_module* ox_module_new(void) { return new ox_module(); }
void ox_module_free(ox_module* m) { delete m; }

ox_module* ox_module_clone(const ox_module* m) {
    auto* c = new ox_module();
    c->b.module() = const_cast<ox_module*>(m)->b.module();
    return c;
}

ox_status ox_module_tp_partition(const ox_module* m, int32_t tp, int32_t rank, ox_module** out) {
    OX_TRY
    auto* c = new ox_module();
    try {
        c->b.module() = tp_partition(const_cast<ox_module*>(m)->b.module(), tp, rank);
    } catch (...) {
        delete c;
        throw;
    }
    *out = c;
    return OX_OK;
    OX_CATCH
}

void ox_module_tp_stats(const ox_module* m, int32_t tp, uint64_t out[3]) {
    size_t c = 0, r = 0, a = 0;
    try {
        tp_partition_stats(const_cast<ox_module*>(m)->b.module(), tp, &c, &r, &a);
    } catch (...) {
    }
    out[0] = c;
    out[1] = r;
    out[2] = a;
}

int32_t ox_module_intern_symbol(ox_module* m, const char* name) {
    return (int32_t)m->b.module().symbols.intern(name);
}

ox_status ox_module_add_const(ox_module* m, int32_t dtype, const uint64_t* dims, int32_t rank, const void* bytes,
                              size_t nbytes, int32_t borrow, int32_t* out_value) {
    OX_TRY
    TensorType ty{dtype_from_c(dtype), fixed_shape(std::vector<uint64_t>(dims, dims + rank))};
    ValueId v;
    if (borrow)
        v = m->b.constant_borrowed(ty, (const uint8_t*)bytes, nbytes);
    else
        v = m->b.constant(ty, std::vector<uint8_t>((const uint8_t*)bytes, (const uint8_t*)bytes + nbytes));
    *out_value = (int32_t)v;
    return OX_OK;
    OX_CATCH
}

ox_status ox_module_add_input(ox_module* m, const char* name, int32_t dtype, const ox_dimexpr* dims, int32_t rank,
                              int32_t* out_value) {
    OX_TRY
    TensorType ty{dtype_from_c(dtype), shape_from_c(dims, rank)};
    *out_value = (int32_t)m->b.input(name, ty);
    return OX_OK;
    OX_CATCH
}

ox_status ox_module_add_prim(ox_module* m, const ox_prim_desc* desc, const int32_t* inputs, int32_t n_in,
                             int32_t* out_value) {
    OX_TRY
    Prim p = prim_from_c(*desc);
    std::vector<ValueId> ins(inputs, inputs + n_in);
    *out_value = (int32_t)m->b.prim(p, ins);
    return OX_OK;
    OX_CATCH
}

ox_status ox_module_add_composite(ox_module* m, const char* name, const ox_attr* attrs, int32_t n_attrs,
                                  const int32_t* inputs, int32_t n_in, const ox_tensor_type* outs, int32_t n_out,
                                  int32_t* out_values) {
    OX_TRY
    Attrs a;
    for (int i = 0; i < n_attrs; i++) {
        const ox_attr& x = attrs[i];
        switch (x.kind) {
            case OX_ATTR_INT: a.set(x.name, AttrValue::of_int(x.i)); break;
            case OX_ATTR_BOOL: a.set(x.name, AttrValue::of_bool(x.i != 0)); break;
            case OX_ATTR_FLOAT: a.set(x.name, AttrValue::of_float(x.f)); break;
            case OX_ATTR_STR: a.set(x.name, AttrValue::of_str(x.s ? x.s : "")); break;
            case OX_ATTR_INTS: a.set(x.name, AttrValue::of_ints(std::vector<int64_t>(x.ints, x.ints + x.n))); break;
            case OX_ATTR_FLOATS: a.set(x.name, AttrValue::of_floats(std::vector<double>(x.floats, x.floats + x.n))); break;
            default: fail(ErrKind::Attribute, std::string("attribute '") + x.name + "': unknown kind");
        }
    }
    std::vector<TensorType> tys;
    for (int i = 0; i < n_out; i++) tys.push_back(TensorType{dtype_from_c(outs[i].dtype), shape_from_c(outs[i].dims, outs[i].rank)});
    std::vector<ValueId> ins(inputs, inputs + n_in);
    auto out = m->b.composite(name, a, ins, tys);
    for (size_t i = 0; i < out.size(); i++) out_values[i] = (int32_t)out[i];
    return OX_OK;
    OX_CATCH
}

ox_status ox_module_add_output(ox_module* m, const char* name, int32_t value) {
    OX_TRY
    m->b.output(name, (ValueId)value);
    return OX_OK;
    OX_CATCH
}

ox_status ox_module_add_constraint(ox_module* m, const ox_dimexpr* left, const ox_dimexpr* right, const char* context) {
    OX_TRY
    m->b.constrain(dim_from_c(*left), dim_from_c(*right), context ? context : "");
    return OX_OK;
    OX_CATCH
}

void ox_module_set_loc(ox_module* m, const char* node_name, const char* op_type) {
    m->b.set_loc(node_name ? std::optional<std::string>(node_name) : std::nullopt,
                 op_type ? std::optional<std::string>(op_type) : std::nullopt);
}

ox_status ox_module_validate(const ox_module* m) {
    OX_TRY
    validate(const_cast<ox_module*>(m)->b.module());
    return OX_OK;
    OX_CATCH
}

ox_status ox_module_inline_composites(ox_module* m, const char* const* keep, int32_t n_keep) {
    OX_TRY
    std::unordered_set<std::string> names;
    for (int i = 0; i < n_keep; i++) names.insert(keep[i]);
    Module out = inline_composites(std::move(m->b.module()), standard_decompositions(),
                                   [&](const Module&, const Node& n) { return names.count(n.composite.name) > 0; });
    m->b.module() = std::move(out);
    return OX_OK;
    OX_CATCH
}

// fold_transpose_into_matmul followed by eliminate_dead; returns 1 when a Transpose was folded, −1 on error.
int32_t ox_module_fold_transposes(ox_module* m) {
    try {
        Module& mod = m->b.module();
        const bool changed = fold_transpose_into_matmul(mod);
        if (changed) eliminate_dead(mod);
        return changed ? 1 : 0;
    } catch (...) {
        return -1;
    }
}

int32_t ox_module_num_nodes(const ox_module* m) { return (int32_t) const_cast<ox_module*>(m)->b.module().nodes.size(); }
int32_t ox_module_num_values(const ox_module* m) { return (int32_t) const_cast<ox_module*>(m)->b.module().values.size(); }
int32_t ox_module_num_inputs(const ox_module* m) { return (int32_t) const_cast<ox_module*>(m)->b.module().inputs.size(); }
int32_t ox_module_num_outputs(const ox_module* m) { return (int32_t) const_cast<ox_module*>(m)->b.module().outputs.size(); }

const char* ox_module_input_name(const ox_module* m, int32_t i) {
    auto& mod = const_cast<ox_module*>(m)->b.module();
    if (i < 0 || (size_t)i >= mod.inputs.size()) return nullptr;
    return mod.inputs[i].first.c_str();
}
const char* ox_module_output_name(const ox_module* m, int32_t i) {
    auto& mod = const_cast<ox_module*>(m)->b.module();
    if (i < 0 || (size_t)i >= mod.outputs.size()) return nullptr;
    return mod.outputs[i].first.c_str();
}

ox_status ox_module_input_desc(const ox_module* m, int32_t i, int32_t* dtype, int32_t* rank) {
    OX_TRY
    auto& mod = const_cast<ox_module*>(m)->b.module();
    if (i < 0 || (size_t)i >= mod.inputs.size()) fail(ErrKind::InvalidGraph, "input index out of range");
    const TensorType& ty = mod.values[mod.inputs[i].second].ty;
    *dtype = (int32_t)ty.dtype;
    *rank = (int32_t)ty.shape.size();
    return OX_OK;
    OX_CATCH
}

ox_status ox_module_eval_input_shape(const ox_module* m, int32_t i, const char* const* sym_names,
                                     const uint64_t* sym_values, int32_t n_syms, uint64_t* out_dims) {
    OX_TRY
    auto& mod = const_cast<ox_module*>(m)->b.module();
    if (i < 0 || (size_t)i >= mod.inputs.size()) fail(ErrKind::InvalidGraph, "input index out of range");
    Bindings b;
    for (int s = 0; s < n_syms; s++)
        if (auto id = mod.symbols.get(sym_names[s])) b.bind(*id, sym_values[s]);
    const TensorType& ty = mod.values[mod.inputs[i].second].ty;
    for (size_t d = 0; d < ty.shape.size(); d++) out_dims[d] = ty.shape[d].eval(b);
    return OX_OK;
    OX_CATCH
}

const char* ox_module_node_op(const ox_module* m, int32_t i) {
    auto& mod = const_cast<ox_module*>(m)->b.module();
    if (i < 0 || (size_t)i >= mod.nodes.size()) return nullptr;
    const Node& n = mod.nodes[i];
    return n.is_prim ? n.prim.name() : n.composite.name.c_str();
}

const char* ox_module_value_type_str(const ox_module* m, int32_t value) {
    static thread_local std::string buf;
    auto& mod = const_cast<ox_module*>(m)->b.module();
    if (value < 0 || (size_t)value >= mod.values.size()) return nullptr;
    buf = mod.values[value].ty.to_string(&mod.symbols);
    return buf.c_str();
}

}  // extern "C"
