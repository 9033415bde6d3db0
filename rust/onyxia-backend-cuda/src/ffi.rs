//! Raw declarations of `include/onyxia_cuda.h`. Field order and widths follow the header exactly.
#![allow(non_camel_case_types, dead_code)]
use std::os::raw::{c_char, c_void};

pub const OX_OK: i32 = 0;
pub const OX_MAX_TERM_SYMS: usize = 6;

// ox_prim_kind
pub const PRIM_UNARY: i32 = 0;
pub const PRIM_BINARY: i32 = 1;
pub const PRIM_COMPARE: i32 = 2;
pub const PRIM_SELECT: i32 = 3;
pub const PRIM_CAST: i32 = 4;
pub const PRIM_MATMUL: i32 = 5;
pub const PRIM_REDUCE: i32 = 6;
pub const PRIM_RESHAPE: i32 = 7;
pub const PRIM_TRANSPOSE: i32 = 8;
pub const PRIM_BROADCAST: i32 = 9;
pub const PRIM_CONCAT: i32 = 10;
pub const PRIM_SLICE: i32 = 11;
pub const PRIM_GATHER: i32 = 12;
pub const PRIM_SCATTER: i32 = 13;
pub const PRIM_IOTA: i32 = 14;
pub const PRIM_DIM_VALUES: i32 = 15;
pub const PRIM_DEQUANTIZE: i32 = 16;

// ox_attr_kind
pub const ATTR_INT: i32 = 0;
pub const ATTR_INTS: i32 = 1;
pub const ATTR_FLOAT: i32 = 2;
pub const ATTR_FLOATS: i32 = 3;
pub const ATTR_STR: i32 = 4;
pub const ATTR_BOOL: i32 = 5;

#[repr(C)]
#[derive(Clone, Copy)]
pub struct ox_dimterm {
    pub coeff: i64,
    pub n_syms: i32,
    pub syms: [i32; OX_MAX_TERM_SYMS],
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct ox_dimexpr {
    pub terms: *const ox_dimterm,
    pub n_terms: i32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct ox_slice_spec {
    pub axis: u64,
    pub start: ox_dimexpr,
    pub end: ox_dimexpr,
    pub step: i64,
}

#[repr(C)]
pub struct ox_prim_desc {
    pub kind: i32,
    pub op: i32,
    pub dtype: i32,
    pub trans_a: i32,
    pub trans_b: i32,
    pub keepdims: i32,
    pub axes: *const u64,
    pub n_axes: i32,
    pub shape: *const ox_dimexpr,
    pub n_shape: i32,
    pub axis: u64,
    pub specs: *const ox_slice_spec,
    pub n_specs: i32,
    pub len: ox_dimexpr,
    pub block_size: u64,
}

#[repr(C)]
pub struct ox_attr {
    pub name: *const c_char,
    pub kind: i32,
    pub i: i64,
    pub f: f64,
    pub s: *const c_char,
    pub ints: *const i64,
    pub floats: *const f64,
    pub n: i32,
}

#[repr(C)]
pub struct ox_tensor_type {
    pub dtype: i32,
    pub dims: *const ox_dimexpr,
    pub rank: i32,
}

#[repr(C)]
#[derive(Default, Clone, Copy)]
pub struct ox_backend_options {
    pub without_fused_kernels: i32,
    pub disable_graphs: i32,
    pub disable_pattern_fusion: i32,
    pub disable_persistent_step: i32,
    pub reserved: [i32; 4],
}

#[repr(C)]
pub struct ox_kernel_timing {
    pub kernel: *const c_char,
    pub node: *const c_char,
    pub time_ns: u64,
}

#[repr(C)]
pub struct ox_module {
    _private: [u8; 0],
}
#[repr(C)]
pub struct ox_backend {
    _private: [u8; 0],
}
#[repr(C)]
pub struct ox_session {
    _private: [u8; 0],
}
#[repr(C)]
pub struct ox_tensor {
    _private: [u8; 0],
}
#[repr(C)]
pub struct ox_llm {
    _private: [u8; 0],
}

unsafe extern "C" {
    pub fn ox_last_error() -> *const c_char;

    pub fn ox_module_new() -> *mut ox_module;
    pub fn ox_module_free(m: *mut ox_module);
    pub fn ox_module_clone(m: *const ox_module) -> *mut ox_module;
    pub fn ox_module_tp_partition(m: *const ox_module, tp: i32, rank: i32, out: *mut *mut ox_module) -> i32;
    pub fn ox_module_tp_stats(m: *const ox_module, tp: i32, out: *mut u64);
    pub fn ox_module_intern_symbol(m: *mut ox_module, name: *const c_char) -> i32;
    pub fn ox_module_add_const(m: *mut ox_module, dtype: i32, dims: *const u64, rank: i32, bytes: *const c_void, nbytes: usize,
                               borrow: i32, out_value: *mut i32) -> i32;
    pub fn ox_module_add_input(m: *mut ox_module, name: *const c_char, dtype: i32, dims: *const ox_dimexpr, rank: i32,
                               out_value: *mut i32) -> i32;
    pub fn ox_module_add_prim(m: *mut ox_module, desc: *const ox_prim_desc, inputs: *const i32, n_in: i32, out_value: *mut i32) -> i32;
    pub fn ox_module_add_composite(m: *mut ox_module, name: *const c_char, attrs: *const ox_attr, n_attrs: i32, inputs: *const i32,
                                   n_in: i32, outs: *const ox_tensor_type, n_out: i32, out_values: *mut i32) -> i32;
    pub fn ox_module_add_output(m: *mut ox_module, name: *const c_char, value: i32) -> i32;
    pub fn ox_module_add_constraint(m: *mut ox_module, left: *const ox_dimexpr, right: *const ox_dimexpr, context: *const c_char) -> i32;
    pub fn ox_module_set_loc(m: *mut ox_module, node_name: *const c_char, op_type: *const c_char);
    pub fn ox_module_fold_transposes(m: *mut ox_module) -> i32;
    pub fn ox_module_validate(m: *const ox_module) -> i32;

    pub fn ox_backend_create(devices: *const i32, n_devices: i32, out: *mut *mut ox_backend) -> i32;
    pub fn ox_backend_create_ex(devices: *const i32, n_devices: i32, options: *const ox_backend_options, out: *mut *mut ox_backend) -> i32;
    pub fn ox_backend_free(b: *mut ox_backend);
    pub fn ox_tp_unique_id(nccl_library_path: *const c_char, out: *mut u8) -> i32;
    pub fn ox_backend_peer_allreduce(b: *const ox_backend) -> i32;
    pub fn ox_backend_join_tp(b: *mut ox_backend, rank: i32, world: i32, id: *const u8, nccl_library_path: *const c_char) -> i32;
    pub fn ox_backend_supports(b: *const ox_backend, composite_name: *const c_char) -> i32;
    pub fn ox_backend_prepare(b: *mut ox_backend, module: *mut ox_module, out: *mut *mut ox_session) -> i32;

    pub fn ox_session_free(s: *mut ox_session);
    pub fn ox_session_upload(s: *mut ox_session, dtype: i32, shape: *const u64, rank: i32, bytes: *const c_void, nbytes: usize,
                             out: *mut *mut ox_tensor) -> i32;
    pub fn ox_session_run(s: *mut ox_session, names: *const *const c_char, inputs: *const *mut ox_tensor, n_in: i32,
                          out_names: *mut *const c_char, out_tensors: *mut *mut ox_tensor, out_cap: i32, n_out: *mut i32) -> i32;
    pub fn ox_session_num_outputs(s: *const ox_session) -> i32;
    pub fn ox_session_download(s: *mut ox_session, t: *const ox_tensor, dst: *mut c_void, cap: usize, written: *mut usize) -> i32;
    pub fn ox_tensor_clone(t: *const ox_tensor) -> *mut ox_tensor;
    pub fn ox_tensor_release(t: *mut ox_tensor);
    pub fn ox_tensor_describe(t: *const ox_tensor, dtype: *mut i32, shape: *mut u64, shape_cap: i32, rank: *mut i32) -> i32;
    pub fn ox_tensor_nbytes(t: *const ox_tensor) -> usize;

    pub fn ox_session_wait_idle(s: *mut ox_session) -> i32;
    pub fn ox_session_resident_bytes(s: *const ox_session) -> u64;
    pub fn ox_session_peak_resident_bytes(s: *const ox_session) -> u64;
    pub fn ox_session_pool_stats(s: *const ox_session, fresh_allocations: *mut u64, reuses: *mut u64);
    pub fn ox_session_enable_profiling(s: *mut ox_session, on: i32) -> i32;
    pub fn ox_session_take_timings(s: *mut ox_session, out: *mut ox_kernel_timing, cap: i32) -> i32;
    pub fn ox_session_launch_count(s: *const ox_session) -> u64;
    pub fn ox_session_argmax_last(s: *mut ox_session, logits: *const ox_tensor, out: *mut *mut ox_tensor) -> i32;
    pub fn ox_session_sample_last(s: *mut ox_session, logits: *const ox_tensor, temperature: f32, top_k: i64, top_p: f32,
                                  uniform: *const f32, n_uniform: usize, out: *mut *mut ox_tensor) -> i32;
    pub fn ox_session_argmax_last_into(s: *mut ox_session, logits: *const ox_tensor, out: *mut ox_tensor) -> i32;

    pub fn ox_llm_create(s: *mut ox_session, max_seq_len: i64, out: *mut *mut ox_llm) -> i32;
    pub fn ox_llm_free(l: *mut ox_llm);
    pub fn ox_llm_sequence_length(l: *const ox_llm) -> i64;
    pub fn ox_llm_logits_dtype(l: *const ox_llm) -> i32;
    pub fn ox_llm_reset(l: *mut ox_llm);
    pub fn ox_llm_step(l: *mut ox_llm, ids: *const i64, n_ids: i32, token_out: *mut i64, logits_out: *mut c_void, logits_cap: usize,
                       logits_written: *mut usize) -> i32;
    pub fn ox_llm_generate(l: *mut ox_llm, ids: *const i64, n_ids: i32, n_new: i32, tokens_out: *mut i64) -> i32;
    pub fn ox_llm_step_sampled(l: *mut ox_llm, ids: *const i64, n_ids: i32, temperature: f32, top_k: i64, top_p: f32, uniform: f32,
                               token_out: *mut i64) -> i32;
}
