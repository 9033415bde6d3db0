//! `onyxia-backend-cuda`: the B200 (sm_100a) execution backend behind the traits of
//! `onyxia_ir::backend` (crates/onyxia-ir/src/backend.rs:24-54), over the C ABI of
//! `libonyxia_cuda.so` (include/onyxia_cuda.h).
//!
//! `prepare` walks the `Module` once and replays it through the C builder calls — symbols,
//! constants (borrowed: the module is alive until `prepare` returns and the library has uploaded
//! them by then), inputs, nodes in order, outputs, constraints — then hands the C module to
//! `ox_backend_prepare`, which legalises it with this backend's kernel registry, plans and uploads.
//! Sessions speak device-resident handles; `run` returns at once with handles whose producers may
//! still be running, `download` waits.
//!
//! The one thing this crate needs from `onyxia-ir` that is not public today is the term list of a
//! `DimExpr` (a polynomial over dimension symbols): `DimExpr::for_each_term(|coeff, syms| …)`, a
//! six-line accessor next to `DimExpr::syms` (crates/onyxia-ir/src/dim.rs:219).
//!
//! Never compiled: there is no Rust toolchain where the native library is developed.

mod ffi;

use std::ffi::{CStr, CString};
use std::os::raw::{c_char, c_void};
use std::ptr;
use std::sync::Arc;

use onyxia_ir::attrs::AttrValue;
use onyxia_ir::backend::{Backend, Session};
use onyxia_ir::graph::{Module, NodeKind, Origin, ValueId};
use onyxia_ir::interp::Tensor;
use onyxia_ir::prim::{Prim, SliceSpec};
use onyxia_ir::{DataType, DimExpr, Error, Result, TensorType};

// ───────────────────────────── errors ───────────────────────────────────

fn last_error() -> String {
    // SAFETY: the library returns a NUL-terminated string owned by the calling thread.
    unsafe {
        let p = ffi::ox_last_error();
        if p.is_null() { String::new() } else { CStr::from_ptr(p).to_string_lossy().into_owned() }
    }
}

/// `ox_status` → `onyxia_ir::Error`, variant for variant (crates/onyxia-ir/src/lib.rs:55-89).
fn check(status: i32) -> Result<()> {
    let msg = || last_error();
    match status {
        0 => Ok(()),
        1 => Err(Error::Shape(msg())),
        2 => Err(Error::InvalidGraph(msg())),
        3 => Err(Error::DType(msg())),
        4 => Err(Error::Attribute(msg())),
        5 => Err(Error::Binding(msg())),
        6 => Err(Error::Interp(msg())),
        7 => Err(Error::Unsupported(msg())),
        _ => Err(Error::Runtime(msg())),
    }
}

fn cstr(s: &str) -> Result<CString> {
    CString::new(s).map_err(|_| Error::InvalidGraph(format!("name with an interior NUL: {s:?}")))
}

fn dtype_code(d: DataType) -> i32 {
    match d {
        DataType::F32 => 0,
        DataType::F16 => 1,
        DataType::I64 => 2,
        DataType::I32 => 3,
        DataType::U32 => 4,
        DataType::U8 => 5,
        DataType::I8 => 6,
        DataType::Bool => 7,
        DataType::U4 => 8,
        DataType::I4 => 9,
    }
}

fn dtype_from_code(c: i32) -> Result<DataType> {
    Ok(match c {
        0 => DataType::F32,
        1 => DataType::F16,
        2 => DataType::I64,
        3 => DataType::I32,
        4 => DataType::U32,
        5 => DataType::U8,
        6 => DataType::I8,
        7 => DataType::Bool,
        8 => DataType::U4,
        9 => DataType::I4,
        _ => return Err(Error::Runtime(format!("unknown dtype code {c} from the backend"))),
    })
}

// ───────────────────────── dimension expressions ────────────────────────

/// Owns the term arrays the `ox_dimexpr` views point into; keep it alive across the call.
#[derive(Default)]
struct DimArena {
    terms: Vec<Vec<ffi::ox_dimterm>>,
}

impl DimArena {
    /// `sym_ids[s.index()]` is the C id of the reference's symbol `s`.
    fn expr(&mut self, e: &DimExpr, sym_ids: &[i32]) -> Result<ffi::ox_dimexpr> {
        let mut terms = Vec::new();
        let mut err = None;
        e.for_each_term(|coeff, syms| {
            if syms.len() > ffi::OX_MAX_TERM_SYMS {
                err = Some(Error::Unsupported(format!("dimension term with {} symbol factors", syms.len())));
                return;
            }
            let mut t = ffi::ox_dimterm { coeff, n_syms: syms.len() as i32, syms: [0; ffi::OX_MAX_TERM_SYMS] };
            for (slot, s) in t.syms.iter_mut().zip(syms) {
                *slot = sym_ids[s.index()];
            }
            terms.push(t);
        });
        if let Some(e) = err {
            return Err(e);
        }
        self.terms.push(terms);
        let stored = self.terms.last().unwrap();
        Ok(ffi::ox_dimexpr { terms: if stored.is_empty() { ptr::null() } else { stored.as_ptr() }, n_terms: stored.len() as i32 })
    }

    fn exprs(&mut self, es: &[DimExpr], sym_ids: &[i32]) -> Result<Vec<ffi::ox_dimexpr>> {
        es.iter().map(|e| self.expr(e, sym_ids)).collect()
    }
}

// ───────────────────────────── backend ──────────────────────────────────

/// ≙ `WgpuBackend` (crates/onyxia-backend-wgpu/src/session.rs:107-242) for CUDA devices.
pub struct CudaBackend {
    raw: *mut ffi::ox_backend,
}

/// Construction options ≙ `ox_backend_options`.
#[derive(Default, Clone, Copy)]
pub struct CudaOptions {
    /// ≙ `WgpuBackend::without_fused_kernels` (session.rs:125-134): every composite runs its decomposition.
    pub without_fused_kernels: bool,
    /// Launch kernels one by one instead of replaying CUDA graphs.
    pub disable_graphs: bool,
    /// Keep every node its own launch (no cross-node fusion).
    pub disable_pattern_fusion: bool,
    /// One launch per operation of a decode step instead of the persistent step kernel.
    pub disable_persistent_step: bool,
}

impl CudaBackend {
    /// A backend on the given CUDA device (one device per backend; several GPUs = one process per GPU joined
    /// into a tensor-parallel group with [`CudaBackend::join_tp`]).
    pub fn new(device: i32) -> Result<Self> {
        Self::with_options(device, CudaOptions::default())
    }

    pub fn with_options(device: i32, o: CudaOptions) -> Result<Self> {
        let opts = ffi::ox_backend_options {
            without_fused_kernels: o.without_fused_kernels as i32,
            disable_graphs: o.disable_graphs as i32,
            disable_pattern_fusion: o.disable_pattern_fusion as i32,
            disable_persistent_step: o.disable_persistent_step as i32,
            reserved: [0; 4],
        };
        let mut raw = ptr::null_mut();
        // SAFETY: plain in/out pointers; `raw` is written only on success.
        check(unsafe { ffi::ox_backend_create_ex(&device, 1, &opts, &mut raw) })?;
        Ok(Self { raw })
    }

    /// ≙ `WgpuBackend::without_fused_kernels`.
    pub fn without_fused_kernels(device: i32) -> Result<Self> {
        Self::with_options(device, CudaOptions { without_fused_kernels: true, ..Default::default() })
    }

    /// The id rank 0 creates and hands to every rank of a new tensor-parallel group (by any channel the host has).
    pub fn tp_unique_id() -> Result<[u8; 128]> {
        let mut id = [0u8; 128];
        check(unsafe { ffi::ox_tp_unique_id(ptr::null(), id.as_mut_ptr()) })?;
        Ok(id)
    }

    /// Joins the group (collective: returns when all `world` ranks have called it). A joined backend executes the
    /// `onyxia.AllReduce` composites of a partitioned module (see [`tp_partition`]).
    pub fn join_tp(&mut self, rank: i32, world: i32, id: &[u8; 128]) -> Result<()> {
        check(unsafe { ffi::ox_backend_join_tp(self.raw, rank, world, id.as_ptr(), ptr::null()) })
    }

    /// Replays `module` through the C builder; returns the C module (owned by the caller).
    fn export(module: &Module) -> Result<*mut ffi::ox_module> {
        struct Guard(*mut ffi::ox_module);
        impl Drop for Guard {
            fn drop(&mut self) {
                if !self.0.is_null() {
                    unsafe { ffi::ox_module_free(self.0) }
                }
            }
        }
        let m = Guard(unsafe { ffi::ox_module_new() });
        if m.0.is_null() {
            return Err(Error::Runtime("ox_module_new failed".into()));
        }

        // symbols, in table order
        let mut sym_ids = Vec::with_capacity(module.symbols.len());
        for name in module.symbols.names() {
            let c = cstr(name)?;
            sym_ids.push(unsafe { ffi::ox_module_intern_symbol(m.0, c.as_ptr()) });
        }

        // values get their C ids as they are created; the walk follows the node order, which is a
        // valid creation order because the reference's builder appends values as it infers them
        let mut c_of: Vec<i32> = vec![-1; module.values.len()];
        let mut arena = DimArena::default();

        let ty_dims = |arena: &mut DimArena, ty: &TensorType| arena.exprs(ty.shape.dims(), &sym_ids);

        // constants and inputs first (they have no producers)
        for (i, def) in module.values.iter().enumerate() {
            match def.origin {
                Origin::Const(cid) => {
                    let ty = module.consts.ty(cid);
                    let dims = ty.shape.as_static().ok_or_else(|| Error::InvalidGraph("constant with a symbolic shape".into()))?;
                    let bytes = module.consts.bytes(cid);
                    let mut out = -1;
                    // the value's own type may be a reinterpretation of the pool entry (graph.rs:230-250): its dtype wins
                    check(unsafe {
                        ffi::ox_module_add_const(m.0, dtype_code(def.ty.dtype), dims.as_ptr(), dims.len() as i32, bytes.as_ptr() as *const c_void,
                                                 bytes.len(), 1 /* borrowed until prepare returns */, &mut out)
                    })?;
                    c_of[i] = out;
                }
                Origin::Input => {}
                Origin::Node { .. } => {}
            }
        }
        for (name, v) in &module.inputs {
            let def = module.value(*v);
            let dims = ty_dims(&mut arena, &def.ty)?;
            let c = cstr(name)?;
            let mut out = -1;
            check(unsafe { ffi::ox_module_add_input(m.0, c.as_ptr(), dtype_code(def.ty.dtype), dims.as_ptr(), dims.len() as i32, &mut out) })?;
            c_of[v.index()] = out;
        }

        let ids_of = |c_of: &[i32], vs: &[ValueId]| -> Result<Vec<i32>> {
            vs.iter()
                .map(|v| match c_of[v.index()] {
                    -1 => Err(Error::InvalidGraph("node reads a value that has not been defined yet".into())),
                    id => Ok(id),
                })
                .collect()
        };

        for nid in module.topo_order()? {
            let node = module.node(nid);
            let loc_name = node.loc.name.as_deref().map(cstr).transpose()?;
            let loc_op = node.loc.op_type.as_deref().map(cstr).transpose()?;
            unsafe {
                ffi::ox_module_set_loc(m.0, loc_name.as_ref().map_or(ptr::null(), |c| c.as_ptr()),
                                       loc_op.as_ref().map_or(ptr::null(), |c| c.as_ptr()))
            };
            let ins = ids_of(&c_of, &node.inputs)?;
            match &node.kind {
                NodeKind::Prim(prim) => {
                    let mut desc = ffi::ox_prim_desc {
                        kind: 0, op: 0, dtype: 0, trans_a: 0, trans_b: 0, keepdims: 0, axes: ptr::null(), n_axes: 0, shape: ptr::null(),
                        n_shape: 0, axis: 0, specs: ptr::null(), n_specs: 0, len: ffi::ox_dimexpr { terms: ptr::null(), n_terms: 0 },
                        block_size: 0,
                    };
                    // buffers the descriptor points into
                    let mut axes: Vec<u64> = Vec::new();
                    let mut shape: Vec<ffi::ox_dimexpr> = Vec::new();
                    let mut specs: Vec<ffi::ox_slice_spec> = Vec::new();
                    match prim {
                        Prim::Unary(op) => {
                            desc.kind = ffi::PRIM_UNARY;
                            desc.op = *op as i32; // declaration order = the header's operator codes (prim.rs:27-107)
                        }
                        Prim::Binary(op) => {
                            desc.kind = ffi::PRIM_BINARY;
                            desc.op = *op as i32;
                        }
                        Prim::Compare(op) => {
                            desc.kind = ffi::PRIM_COMPARE;
                            desc.op = *op as i32;
                        }
                        Prim::Select => desc.kind = ffi::PRIM_SELECT,
                        Prim::Cast { to } => {
                            desc.kind = ffi::PRIM_CAST;
                            desc.dtype = dtype_code(*to);
                        }
                        Prim::MatMul { trans_a, trans_b } => {
                            desc.kind = ffi::PRIM_MATMUL;
                            desc.trans_a = *trans_a as i32;
                            desc.trans_b = *trans_b as i32;
                        }
                        Prim::Reduce { op, axes: a, keepdims } => {
                            desc.kind = ffi::PRIM_REDUCE;
                            desc.op = *op as i32;
                            desc.keepdims = *keepdims as i32;
                            axes = a.iter().map(|&x| x as u64).collect();
                        }
                        Prim::Reshape { shape: s } => {
                            desc.kind = ffi::PRIM_RESHAPE;
                            shape = arena.exprs(s, &sym_ids)?;
                        }
                        Prim::Transpose { perm } => {
                            desc.kind = ffi::PRIM_TRANSPOSE;
                            axes = perm.iter().map(|&x| x as u64).collect();
                        }
                        Prim::Broadcast { shape: s } => {
                            desc.kind = ffi::PRIM_BROADCAST;
                            shape = arena.exprs(s, &sym_ids)?;
                        }
                        Prim::Concat { axis } => {
                            desc.kind = ffi::PRIM_CONCAT;
                            desc.axis = *axis as u64;
                        }
                        Prim::Slice { specs: ss } => {
                            desc.kind = ffi::PRIM_SLICE;
                            for SliceSpec { axis, start, end, step } in ss {
                                specs.push(ffi::ox_slice_spec {
                                    axis: *axis as u64,
                                    start: arena.expr(start, &sym_ids)?,
                                    end: arena.expr(end, &sym_ids)?,
                                    step: *step,
                                });
                            }
                        }
                        Prim::Gather { axis } => {
                            desc.kind = ffi::PRIM_GATHER;
                            desc.axis = *axis as u64;
                        }
                        Prim::Scatter => desc.kind = ffi::PRIM_SCATTER,
                        Prim::Iota { len, dtype } => {
                            desc.kind = ffi::PRIM_IOTA;
                            desc.len = arena.expr(len, &sym_ids)?;
                            desc.dtype = dtype_code(*dtype);
                        }
                        Prim::DimValues { exprs } => {
                            desc.kind = ffi::PRIM_DIM_VALUES;
                            shape = arena.exprs(exprs, &sym_ids)?;
                        }
                        Prim::Dequantize { block_size, out_shape } => {
                            desc.kind = ffi::PRIM_DEQUANTIZE;
                            desc.block_size = *block_size as u64;
                            shape = arena.exprs(out_shape, &sym_ids)?;
                        }
                    }
                    desc.axes = if axes.is_empty() { ptr::null() } else { axes.as_ptr() };
                    desc.n_axes = axes.len() as i32;
                    desc.shape = if shape.is_empty() { ptr::null() } else { shape.as_ptr() };
                    desc.n_shape = shape.len() as i32;
                    desc.specs = if specs.is_empty() { ptr::null() } else { specs.as_ptr() };
                    desc.n_specs = specs.len() as i32;
                    let mut out = -1;
                    check(unsafe { ffi::ox_module_add_prim(m.0, &desc, ins.as_ptr(), ins.len() as i32, &mut out) })?;
                    c_of[node.outputs[0].index()] = out;
                }
                NodeKind::Composite(comp) => {
                    let name = cstr(&comp.name)?;
                    // attribute storage the ox_attr views point into
                    let mut names = Vec::new();
                    let mut strs = Vec::new();
                    let mut attrs = Vec::new();
                    for (an, av) in comp.attrs.iter() {
                        names.push(cstr(an)?);
                        let mut a = ffi::ox_attr {
                            name: names.last().unwrap().as_ptr(), kind: 0, i: 0, f: 0.0, s: ptr::null(), ints: ptr::null(), floats: ptr::null(), n: 0,
                        };
                        match av {
                            AttrValue::Int(v) => {
                                a.kind = ffi::ATTR_INT;
                                a.i = *v;
                            }
                            AttrValue::Bool(v) => {
                                a.kind = ffi::ATTR_BOOL;
                                a.i = *v as i64;
                            }
                            AttrValue::Float(v) => {
                                a.kind = ffi::ATTR_FLOAT;
                                a.f = *v;
                            }
                            AttrValue::Ints(v) => {
                                a.kind = ffi::ATTR_INTS;
                                a.ints = v.as_ptr();
                                a.n = v.len() as i32;
                            }
                            AttrValue::Floats(v) => {
                                a.kind = ffi::ATTR_FLOATS;
                                a.floats = v.as_ptr();
                                a.n = v.len() as i32;
                            }
                            AttrValue::Str(v) => {
                                a.kind = ffi::ATTR_STR;
                                strs.push(cstr(v)?);
                                a.s = strs.last().unwrap().as_ptr();
                            }
                            AttrValue::Tensor(_) => {
                                return Err(Error::Unsupported(format!("tensor-valued attribute '{an}' on composite '{}'", comp.name)));
                            }
                        }
                        attrs.push(a);
                    }
                    let mut out_dims: Vec<Vec<ffi::ox_dimexpr>> = Vec::new();
                    for v in &node.outputs {
                        out_dims.push(ty_dims(&mut arena, &module.value(*v).ty)?);
                    }
                    let outs: Vec<ffi::ox_tensor_type> = node
                        .outputs
                        .iter()
                        .zip(&out_dims)
                        .map(|(v, d)| ffi::ox_tensor_type { dtype: dtype_code(module.value(*v).ty.dtype), dims: d.as_ptr(), rank: d.len() as i32 })
                        .collect();
                    let mut out_ids = vec![-1i32; outs.len()];
                    check(unsafe {
                        ffi::ox_module_add_composite(m.0, name.as_ptr(), attrs.as_ptr(), attrs.len() as i32, ins.as_ptr(), ins.len() as i32,
                                                     outs.as_ptr(), outs.len() as i32, out_ids.as_mut_ptr())
                    })?;
                    for (v, id) in node.outputs.iter().zip(out_ids) {
                        c_of[v.index()] = id;
                    }
                }
            }
        }
        unsafe { ffi::ox_module_set_loc(m.0, ptr::null(), ptr::null()) };

        for (name, v) in &module.outputs {
            let c = cstr(name)?;
            check(unsafe { ffi::ox_module_add_output(m.0, c.as_ptr(), c_of[v.index()]) })?;
        }
        for con in &module.constraints {
            let (l, r) = (arena.expr(&con.left, &sym_ids)?, arena.expr(&con.right, &sym_ids)?);
            let ctx = cstr(&con.context)?;
            check(unsafe { ffi::ox_module_add_constraint(m.0, &l, &r, ctx.as_ptr()) })?;
        }
        let raw = m.0;
        std::mem::forget(m);
        Ok(raw)
    }
}

impl Drop for CudaBackend {
    fn drop(&mut self) {
        unsafe { ffi::ox_backend_free(self.raw) }
    }
}

impl Backend for CudaBackend {
    type Session = CudaSession;

    fn supports(&self, composite: &str) -> bool {
        match CString::new(composite) {
            Ok(c) => unsafe { ffi::ox_backend_supports(self.raw, c.as_ptr()) != 0 },
            Err(_) => false,
        }
    }

    fn prepare(&self, module: Module) -> Result<CudaSession> {
        let c_module = Self::export(&module)?;
        let mut raw = ptr::null_mut();
        // consumes `c_module`, also on failure; the borrowed constants have been uploaded when it returns
        check(unsafe { ffi::ox_backend_prepare(self.raw, c_module, &mut raw) })?;
        drop(module); // only now may the host copy of the weights go
        Ok(CudaSession { raw })
    }
}

/// The per-rank module of a tensor-parallel group ≙ `ox_module_tp_partition`: column-split Q/K/V/gate/up,
/// row-split O/down, one `onyxia.AllReduce` after the attention block and one after the FFN block. Returned
/// as a prepared session because the partition exists only on the C side.
pub fn prepare_tp(backend: &CudaBackend, module: Module, tp: i32, rank: i32) -> Result<CudaSession> {
    let whole = CudaBackend::export(&module)?;
    let mut part = ptr::null_mut();
    let st = unsafe { ffi::ox_module_tp_partition(whole, tp, rank, &mut part) };
    unsafe { ffi::ox_module_free(whole) };
    check(st)?;
    let mut raw = ptr::null_mut();
    check(unsafe { ffi::ox_backend_prepare(backend.raw, part, &mut raw) })?;
    drop(module);
    Ok(CudaSession { raw })
}

// ───────────────────────────── session ──────────────────────────────────

struct Handle(*mut ffi::ox_tensor);
impl Drop for Handle {
    fn drop(&mut self) {
        unsafe { ffi::ox_tensor_release(self.0) }
    }
}

/// Device-resident tensor handle ≙ `GpuTensor` (session.rs:23-30): cheap to clone, may outlive the session
/// that produced it, may be fed to a later `run`.
#[derive(Clone)]
pub struct CudaTensor(Arc<Handle>);

impl CudaTensor {
    fn raw(&self) -> *mut ffi::ox_tensor {
        self.0.0
    }

    pub fn describe(&self) -> Result<(DataType, Vec<usize>)> {
        let (mut dt, mut rank) = (0i32, 0i32);
        let mut shape = [0u64; 8];
        check(unsafe { ffi::ox_tensor_describe(self.raw(), &mut dt, shape.as_mut_ptr(), 8, &mut rank) })?;
        Ok((dtype_from_code(dt)?, shape[..rank as usize].iter().map(|&d| d as usize).collect()))
    }
}

pub struct CudaSession {
    raw: *mut ffi::ox_session,
}

impl Drop for CudaSession {
    fn drop(&mut self) {
        unsafe { ffi::ox_session_free(self.raw) }
    }
}

impl CudaSession {
    /// ≙ `WgpuSession::wait_idle` (session.rs:280-340); also surfaces execution errors of earlier runs.
    pub fn wait_idle(&mut self) -> Result<()> {
        check(unsafe { ffi::ox_session_wait_idle(self.raw) })
    }
    pub fn resident_bytes(&self) -> u64 {
        unsafe { ffi::ox_session_resident_bytes(self.raw) }
    }
    pub fn peak_resident_bytes(&self) -> u64 {
        unsafe { ffi::ox_session_peak_resident_bytes(self.raw) }
    }
    /// Greedy choice on the device ≙ `sample_greedy` (crates/onyxia-cli/src/sampling.rs:71-80): the last of equal maxima.
    pub fn argmax_last(&mut self, logits: &CudaTensor) -> Result<CudaTensor> {
        let mut out = ptr::null_mut();
        check(unsafe { ffi::ox_session_argmax_last(self.raw, logits.raw(), &mut out) })?;
        Ok(CudaTensor(Arc::new(Handle(out))))
    }
    /// Temperature / top-k / top-p choice on the device ≙ `sample` (crates/onyxia-cli/src/sampling.rs:36-65). The caller
    /// keeps the generator: `uniform` holds one `next_u32() as f32 / u32::MAX as f32` per row of the logits.
    pub fn sample_last(&mut self, logits: &CudaTensor, temperature: f32, top_k: usize, top_p: f32, uniform: &[f32]) -> Result<CudaTensor> {
        let mut out = ptr::null_mut();
        check(unsafe {
            ffi::ox_session_sample_last(self.raw, logits.raw(), temperature, top_k as i64, top_p, uniform.as_ptr(), uniform.len(), &mut out)
        })?;
        Ok(CudaTensor(Arc::new(Handle(out))))
    }
}

#[async_trait::async_trait(?Send)]
impl Session for CudaSession {
    type Tensor = CudaTensor;

    fn upload(&mut self, tensor: &Tensor) -> Result<CudaTensor> {
        let shape: Vec<u64> = tensor.shape().iter().map(|&d| d as u64).collect();
        let bytes = tensor.bytes();
        let mut out = ptr::null_mut();
        check(unsafe {
            ffi::ox_session_upload(self.raw, dtype_code(tensor.dtype()), shape.as_ptr(), shape.len() as i32, bytes.as_ptr() as *const c_void,
                                   bytes.len(), &mut out)
        })?;
        Ok(CudaTensor(Arc::new(Handle(out))))
    }

    async fn run(&mut self, inputs: &[(&str, CudaTensor)]) -> Result<Vec<(String, CudaTensor)>> {
        let names: Vec<CString> = inputs.iter().map(|(n, _)| cstr(n)).collect::<Result<_>>()?;
        let name_ptrs: Vec<*const c_char> = names.iter().map(|c| c.as_ptr()).collect();
        let tensors: Vec<*mut ffi::ox_tensor> = inputs.iter().map(|(_, t)| t.raw()).collect();
        let cap = unsafe { ffi::ox_session_num_outputs(self.raw) }.max(0) as usize;
        let mut out_names: Vec<*const c_char> = vec![ptr::null(); cap];
        let mut out_tensors: Vec<*mut ffi::ox_tensor> = vec![ptr::null_mut(); cap];
        let mut n_out = 0i32;
        check(unsafe {
            ffi::ox_session_run(self.raw, name_ptrs.as_ptr(), tensors.as_ptr(), inputs.len() as i32, out_names.as_mut_ptr(),
                                out_tensors.as_mut_ptr(), cap as i32, &mut n_out)
        })?;
        let mut outs = Vec::with_capacity(n_out as usize);
        for i in 0..n_out as usize {
            // names point into session-owned storage: copy them out
            let name = unsafe { CStr::from_ptr(out_names[i]) }.to_string_lossy().into_owned();
            outs.push((name, CudaTensor(Arc::new(Handle(out_tensors[i])))));
        }
        Ok(outs)
    }

    async fn download(&mut self, tensor: &CudaTensor) -> Result<Tensor> {
        let (dtype, shape) = tensor.describe()?;
        let nbytes = unsafe { ffi::ox_tensor_nbytes(tensor.raw()) };
        let mut data = vec![0u8; nbytes];
        let mut written = 0usize;
        check(unsafe { ffi::ox_session_download(self.raw, tensor.raw(), data.as_mut_ptr() as *mut c_void, nbytes, &mut written) })?;
        data.truncate(written);
        Tensor::new(dtype, shape, data)
    }
}

// ───────────────────────── native generation loop ───────────────────────

/// `LlmSession` (crates/onyxia-cli/src/llm.rs:26-246) as one library call per step: present → past feedback,
/// all-ones masks and the greedy choice happen inside the library; 8 + 8·T bytes go up and 8 bytes come back
/// per decoded token. The generic `LlmSession<B>` keeps working over [`CudaBackend`]; this is the fast path.
pub struct CudaLlm<'s> {
    raw: *mut ffi::ox_llm,
    _session: &'s mut CudaSession,
}

impl<'s> CudaLlm<'s> {
    pub fn new(session: &'s mut CudaSession, max_seq_len: i64) -> Result<Self> {
        let mut raw = ptr::null_mut();
        check(unsafe { ffi::ox_llm_create(session.raw, max_seq_len, &mut raw) })?;
        Ok(Self { raw, _session: session })
    }
    /// Runs `ids` (a prompt, or one token) and returns the greedy next token.
    pub fn step_greedy(&mut self, ids: &[i64]) -> Result<i64> {
        let mut tok = 0i64;
        check(unsafe { ffi::ox_llm_step(self.raw, ids.as_ptr(), ids.len() as i32, &mut tok, ptr::null_mut(), 0, ptr::null_mut()) })?;
        Ok(tok)
    }
    /// `n_new` greedy tokens after `ids`, the token id passed from step to step on the device.
    pub fn generate(&mut self, ids: &[i64], n_new: usize) -> Result<Vec<i64>> {
        let mut out = vec![0i64; n_new];
        check(unsafe { ffi::ox_llm_generate(self.raw, ids.as_ptr(), ids.len() as i32, n_new as i32, out.as_mut_ptr()) })?;
        Ok(out)
    }
    /// The same step with the next token drawn on the device ≙ `sample` (crates/onyxia-cli/src/sampling.rs:36-65);
    /// `uniform` is `rng.next_u32() as f32 / u32::MAX as f32` from the caller's generator.
    pub fn step_sampled(&mut self, ids: &[i64], temperature: f32, top_k: usize, top_p: f32, uniform: f32) -> Result<i64> {
        let mut tok = 0i64;
        check(unsafe { ffi::ox_llm_step_sampled(self.raw, ids.as_ptr(), ids.len() as i32, temperature, top_k as i64, top_p, uniform, &mut tok) })?;
        Ok(tok)
    }
    pub fn sequence_length(&self) -> i64 {
        unsafe { ffi::ox_llm_sequence_length(self.raw) }
    }
    pub fn reset(&mut self) {
        unsafe { ffi::ox_llm_reset(self.raw) }
    }
}

impl Drop for CudaLlm<'_> {
    fn drop(&mut self) {
        unsafe { ffi::ox_llm_free(self.raw) }
    }
}
