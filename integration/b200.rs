//! B200 backend for rai: the Rust side of the drop-in, to be added to the rai tree as
//! `rai-core/src/backend/b200.rs` behind a Cargo feature `b200`.
//!
//! STATUS: this file has never been compiled.  The environment it was written in has no Rust toolchain
//! (no cargo, no rustc), so it is source for a rai maintainer to build, written against the interfaces of
//! rai v0.11.0 as they appear in its tree:
//!   - `trait Backend`, `trait Eval<D, P>`                     rai-core/src/backend/mod.rs:8-13,48-54
//!   - `trait TensorLike`                                      rai-core/src/tensor.rs:19-26
//!   - `Tensor::get_data / set_data`                           rai-core/src/tensor.rs:151-179
//!   - `dispatch::register::<D, P, B>(backend)`                rai-core/src/dispatch.rs:181-189
//!   - the rule set `register_backend!` installs               rai-core/src/dispatch.rs:41-157
//!   - the reference rules it replaces                         rai-core/src/backend/candle.rs:197-1004
//! The library side (librai_b200.so, C ABI in include/rai_b200.h) is what the repository builds and tests.
//!
//! Wiring (three small edits outside this file):
//!   rai-core/Cargo.toml     [features] b200 = []                     (next to `cuda`, rai-core/Cargo.toml:30-39)
//!   rai-core/build.rs       println!("cargo:rustc-link-search=native={}", env!("RAI_B200_LIB_DIR"));
//!                           println!("cargo:rustc-link-lib=dylib=rai_b200");
//!   rai-core/src/backend/mod.rs   #[cfg(feature = "b200")] pub mod b200;
//! and one call at program start: `rai::backend::b200::register_all();` — it overwrites the `(Cuda, op)` keys of
//! the dispatch table (dispatch.rs:191-204 inserts, so a later registration wins).
//!
//! Storage model.  The reference's storage is `candle_core::Tensor` (an Arc'd buffer plus a layout), so views are
//! free and kernels see strides.  `B200Tensor` does the same: an `Rc<Allocation>` shared by all views of one
//! buffer, an element offset, a shape and strides.  View ops (Narrow, Transpose, Permute, Reshape of a dense
//! tensor, Broadcast) only build a new `B200Tensor`; kernels that need dense operands call `dense()`, which copies
//! through `rb_copy_strided` when the view is not already dense.  Allocations come from the library's
//! stream-ordered pool (`rb_malloc_async` / `rb_free_async`), so allocating an output per node — what every
//! reference rule does — costs no device synchronisation.
//!
//! Errors.  `Eval::eval` returns `()`; the reference unwraps candle's errors, so a failing rule panics.  `check`
//! does the same with the library's status and `rb_last_error()` text.

#![allow(non_camel_case_types, clippy::missing_safety_doc)]

use crate::{
    dispatch, ops, Backend, Cpu, Cuda, DType, Eval, Tensor, TensorLike, Type, BF16, F16, F32, F64, I64, U32, U8,
};
use half::{bf16, f16};
use once_cell::sync::Lazy;
use std::{
    any::{Any, TypeId},
    collections::HashMap,
    ffi::{c_char, c_void, CStr},
    fmt,
    ops::Deref,
    rc::Rc,
    sync::RwLock,
};

// ------------------------------------------------------------------------------------------------ FFI
#[repr(C)]
pub struct rb_ctx {
    _p: [u8; 0],
}
#[repr(C)]
pub struct rb_kv_cache {
    _p: [u8; 0],
}
#[repr(C)]
pub struct rb_model {
    _p: [u8; 0],
}
#[repr(C)]
pub struct rb_safetensors {
    _p: [u8; 0],
}
/// `struct rb_model_config` of include/rai_b200.h, field for field.
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct rb_model_config {
    pub arch: i32,
    pub dtype: i32,
    pub vocab_size: i32,
    pub hidden_size: i32,
    pub intermediate_size: i32,
    pub num_hidden_layers: i32,
    pub num_attention_heads: i32,
    pub num_key_value_heads: i32,
    pub max_position_embeddings: i32,
    pub rotary_dim: i32,
    pub hidden_act: i32,
    pub tie_word_embeddings: i32,
    pub max_batch: i32,
    pub max_seq: i32,
    pub max_tokens: i32,
    pub tp_rank: i32,
    pub tp_size: i32,
    pub sliding_window: i32,
    pub reserved0: i32,
    pub rope_theta: f64,
    pub norm_eps: f64,
}

// Every entry point of include/rai_b200.h.  The block between the markers is emitted by
// integration/gen_ffi.py from the header and checked against it by tests/test_abi.py.
// <ffi>
extern "C" {
    pub fn rb_init(device: i32, out: *mut *mut rb_ctx) -> i32;
    pub fn rb_destroy(ctx: *mut rb_ctx) -> i32;
    pub fn rb_set_stream(ctx: *mut rb_ctx, cuda_stream: *mut c_void) -> i32;
    pub fn rb_sync(ctx: *mut rb_ctx) -> i32;
    pub fn rb_last_error() -> *const c_char;
    pub fn rb_status_word(ctx: *mut rb_ctx, out4: *mut u32) -> i32;
    pub fn rb_sm_count(ctx: *mut rb_ctx) -> i32;
    pub fn rb_set_wait_budget_us(ctx: *mut rb_ctx, microseconds: i64) -> i32;
    pub fn rb_selftest_wait_gives_up(ctx: *mut rb_ctx, which: i32, budget_us: i64) -> i32;
    pub fn rb_malloc(ctx: *mut rb_ctx, bytes: usize, out_dev: *mut *mut c_void) -> i32;
    pub fn rb_free(ctx: *mut rb_ctx, dev: *mut c_void) -> i32;
    pub fn rb_malloc_async(ctx: *mut rb_ctx, bytes: usize, out_dev: *mut *mut c_void) -> i32;
    pub fn rb_free_async(ctx: *mut rb_ctx, dev: *mut c_void) -> i32;
    pub fn rb_upload(ctx: *mut rb_ctx, dst_dev: *mut c_void, src_host: *const c_void, bytes: usize) -> i32;
    pub fn rb_download(ctx: *mut rb_ctx, dst_host: *mut c_void, src_dev: *const c_void, bytes: usize) -> i32;
    pub fn rb_embed_gather(ctx: *mut rb_ctx, table_dev: *const c_void, dtype: i32, vocab: i64, hidden: i64, ids_dev: *const u32, n_ids: i64, scale: f32, out_dev: *mut c_void) -> i32;
    pub fn rb_norm(ctx: *mut rb_ctx, kind: i32, x_dev: *const c_void, add_dev: *const c_void, acc_dev: *const f32, n_acc: i32, acc_bias_dev: *const c_void, weight_dev: *const c_void, bias_dev: *const c_void, eps: f32, rows: i64, hidden: i64, out_dev: *mut c_void, sum_out_dev: *mut c_void, dtype: i32) -> i32;
    pub fn rb_linear(ctx: *mut rb_ctx, x_dev: *const c_void, w_dev: *const c_void, bias_dev: *const c_void, residual_dev: *const c_void, out_dev: *mut c_void, m: i64, n: i64, k: i64, act: i32, dtype: i32) -> i32;
    pub fn rb_gated_linear(ctx: *mut rb_ctx, x_dev: *const c_void, wg_dev: *const c_void, wu_dev: *const c_void, out_dev: *mut c_void, m: i64, n: i64, k: i64, act: i32, dtype: i32) -> i32;
    pub fn rb_linear_partials(ctx: *mut rb_ctx, x_dev: *const c_void, w_dev: *const c_void, part_dev: *mut f32, m: i64, n: i64, k: i64, n_split: i32) -> i32;
    pub fn rb_linear_pick_splits(ctx: *mut rb_ctx, m: i64, n: i64, k: i64) -> i32;
    pub fn rb_kv_cache_create(ctx: *mut rb_ctx, layers: i32, kv_heads: i32, head_dim: i32, max_batch: i32, max_seq: i32, dtype: i32, out: *mut *mut rb_kv_cache) -> i32;
    pub fn rb_kv_cache_destroy(c: *mut rb_kv_cache) -> i32;
    pub fn rb_kv_cache_reset(c: *mut rb_kv_cache) -> i32;
    pub fn rb_kv_cache_set_window(c: *mut rb_kv_cache, window: i32) -> i32;
    pub fn rb_kv_cache_set_len(c: *mut rb_kv_cache, batch: i32, len: i32) -> i32;
    pub fn rb_kv_cache_read(c: *mut rb_kv_cache, layer: i32, seq: i32, kv_head: i32, t0: i32, n: i32, k_host: *mut c_void, v_host: *mut c_void) -> i32;
    pub fn rb_rope_tables(ctx: *mut rb_ctx, recipe: i32, rot_dim: i32, max_pos: i32, theta: f64, cos_dev: *mut f32, sin_dev: *mut f32) -> i32;
    pub fn rb_rope_kv_append(ctx: *mut rb_ctx, qkv_dev: *const c_void, acc_dev: *const f32, n_acc: i32, bias_dev: *const c_void, cos_dev: *const f32, sin_dev: *const f32, rot_dim: i32, batch: i32, s_new: i32, q_heads: i32, cache: *mut rb_kv_cache, layer: i32, q_out_dev: *mut c_void, dtype: i32) -> i32;
    pub fn rb_attention(ctx: *mut rb_ctx, q_dev: *const c_void, cache: *mut rb_kv_cache, layer: i32, batch: i32, s_new: i32, q_heads: i32, scale: f32, out_dev: *mut c_void, dtype: i32) -> i32;
    pub fn rb_attention_decode_static(ctx: *mut rb_ctx, q_dev: *const c_void, cache: *mut rb_kv_cache, layer: i32, batch: i32, q_heads: i32, scale: f32, out_dev: *mut c_void) -> i32;
    pub fn rb_rope_attention_decode(ctx: *mut rb_ctx, qkv_dev: *const c_void, acc_dev: *const f32, n_acc: i32, bias_dev: *const c_void, cos_dev: *const f32, sin_dev: *const f32, rot: i32, batch: i32, q_heads: i32, cache: *mut rb_kv_cache, layer: i32, scale: f32, q_scratch_dev: *mut c_void, out_dev: *mut c_void, dtype: i32) -> i32;
    pub fn rb_argmax_rows(ctx: *mut rb_ctx, logits_dev: *const c_void, dtype: i32, rows: i64, cols: i64, out_dev: *mut u32) -> i32;
    pub fn rb_sample_greedy(ctx: *mut rb_ctx, logits_dev: *const c_void, dtype: i32, rows: i64, cols: i64, penalty: f32, context_dev: *const i32, context_stride: i32, context_count_dev: *const i32, eos_token: i32, finished_dev: *mut u8, out_dev: *mut u32) -> i32;
    pub fn rb_unary(ctx: *mut rb_ctx, op: i32, x_dev: *const c_void, out_dev: *mut c_void, n: i64, scalar: f32, dtype: i32) -> i32;
    pub fn rb_binary(ctx: *mut rb_ctx, op: i32, a_dev: *const c_void, a_strides: *const i64, b_dev: *const c_void, b_strides: *const i64, out_dev: *mut c_void, rank: i32, shape: *const i64, dtype: i32) -> i32;
    pub fn rb_softmax_rows(ctx: *mut rb_ctx, x_dev: *const c_void, out_dev: *mut c_void, rows: i64, cols: i64, dtype: i32) -> i32;
    pub fn rb_reduce_rows(ctx: *mut rb_ctx, op: i32, x_dev: *const c_void, out_dev: *mut c_void, rows: i64, cols: i64, dtype: i32) -> i32;
    pub fn rb_copy_strided(ctx: *mut rb_ctx, x_dev: *const c_void, x_strides: *const i64, x_offset: i64, out_dev: *mut c_void, out_strides: *const i64, out_offset: i64, rank: i32, shape: *const i64, elem_size: i32) -> i32;
    pub fn rb_cast(ctx: *mut rb_ctx, x_dev: *const c_void, src_dtype: i32, out_dev: *mut c_void, dst_dtype: i32, n: i64) -> i32;
    pub fn rb_index_select(ctx: *mut rb_ctx, x_dev: *const c_void, outer: i64, dim: i64, inner: i64, idx_dev: *const u32, n_idx: i64, out_dev: *mut c_void, elem_size: i32) -> i32;
    pub fn rb_gather_last(ctx: *mut rb_ctx, x_dev: *const c_void, rows: i64, cols: i64, idx_dev: *const u32, k: i64, out_dev: *mut c_void, elem_size: i32) -> i32;
    pub fn rb_where(ctx: *mut rb_ctx, cond_dev: *const u8, on_true_dev: *const c_void, on_false_dev: *const c_void, out_dev: *mut c_void, n: i64, dtype: i32) -> i32;
    pub fn rb_fill(ctx: *mut rb_ctx, out_dev: *mut c_void, n: i64, value: f64, dtype: i32) -> i32;
    pub fn rb_arange(ctx: *mut rb_ctx, out_dev: *mut c_void, n: i64, start: f64, step: f64, dtype: i32) -> i32;
    pub fn rb_matmul(ctx: *mut rb_ctx, a_dev: *const c_void, b_dev: *const c_void, c_dev: *mut c_void, batch: i64, m: i64, n: i64, k: i64, a_batch_stride: i64, b_batch_stride: i64, trans_b: i32, dtype: i32) -> i32;
    pub fn rb_compare(ctx: *mut rb_ctx, op: i32, a_dev: *const c_void, a_strides: *const i64, b_dev: *const c_void, b_strides: *const i64, out_dev: *mut u8, rank: i32, shape: *const i64, dtype: i32) -> i32;
    pub fn rb_log_softmax_rows(ctx: *mut rb_ctx, x_dev: *const c_void, out_dev: *mut c_void, rows: i64, cols: i64, dtype: i32) -> i32;
    pub fn rb_argmin_rows(ctx: *mut rb_ctx, x_dev: *const c_void, dtype: i32, rows: i64, cols: i64, out_dev: *mut u32) -> i32;
    pub fn rb_scatter_add(ctx: *mut rb_ctx, x_dev: *const c_void, src_dev: *const c_void, idx_dev: *const u32, out_dev: *mut c_void, outer: i64, dim_out: i64, dim_src: i64, inner: i64, index_is_1d: i32, dtype: i32) -> i32;
    pub fn rb_conv2d(ctx: *mut rb_ctx, x_dev: *const c_void, x_shape4: *const i32, w_dev: *const c_void, w_shape4: *const i32, padding2: *const i32, stride2: *const i32, dilation2: *const i32, out_dev: *mut c_void, out_shape4: *mut i32, dtype: i32) -> i32;
    pub fn rb_conv_transpose2d(ctx: *mut rb_ctx, x_dev: *const c_void, x_shape4: *const i32, w_dev: *const c_void, w_shape4: *const i32, padding2: *const i32, out_padding2: *const i32, stride2: *const i32, dilation2: *const i32, out_dev: *mut c_void, out_shape4: *mut i32, dtype: i32) -> i32;
    pub fn rb_pool2d(ctx: *mut rb_ctx, is_max: i32, x_dev: *const c_void, x_shape4: *const i32, kernel2: *const i32, stride2: *const i32, padding2: *const i32, dilation2: *const i32, out_dev: *mut c_void, out_shape4: *mut i32, dtype: i32) -> i32;
    pub fn rb_upsample_nearest2d(ctx: *mut rb_ctx, x_dev: *const c_void, x_shape4: *const i32, out_h: i32, out_w: i32, out_dev: *mut c_void, dtype: i32) -> i32;
    pub fn rb_model_create(ctx: *mut rb_ctx, cfg: *const rb_model_config, out: *mut *mut rb_model) -> i32;
    pub fn rb_model_destroy(m: *mut rb_model) -> i32;
    pub fn rb_model_load_param(m: *mut rb_model, name: *const c_char, data: *const c_void, on_device: i32, src_dtype: i32, rank: i32, shape: *const i64) -> i32;
    pub fn rb_model_read_param(m: *mut rb_model, name: *const c_char, dst_host: *mut c_void, dst_bytes: usize) -> i32;
    pub fn rb_model_load_safetensors(m: *mut rb_model, paths: *const *const c_char, n_paths: i32) -> i32;
    pub fn rb_safetensors_open(path: *const c_char, out: *mut *mut rb_safetensors) -> i32;
    pub fn rb_safetensors_close(st: *mut rb_safetensors) -> i32;
    pub fn rb_safetensors_count(st: *const rb_safetensors) -> i32;
    pub fn rb_safetensors_entry(st: *const rb_safetensors, index: i32, name: *mut *const c_char, dtype: *mut i32, rank: *mut i32, shape8: *mut i64, data: *mut *const c_void, bytes: *mut u64) -> i32;
    pub fn rb_model_finalize(m: *mut rb_model) -> i32;
    pub fn rb_model_param_count(m: *mut rb_model) -> i32;
    pub fn rb_model_param_name(m: *mut rb_model, i: i32) -> *const c_char;
    pub fn rb_model_tp_init(m: *mut rb_model, nccl_id: *const c_void, id_bytes: i32) -> i32;
    pub fn rb_tp_unique_id(out128: *mut c_void) -> i32;
    pub fn rb_model_forward(m: *mut rb_model, tokens_dev: *const u32, batch: i32, seq: i32, pos: i32, logits_dev: *mut c_void) -> i32;
    pub fn rb_model_forward_ragged(m: *mut rb_model, tokens_dev: *const u32, batch: i32, seq: i32, pos: i32, lens_host: *const i32, logits_dev: *mut c_void) -> i32;
    pub fn rb_model_generate_ragged(m: *mut rb_model, tokens_host: *const u32, batch: i32, seq: i32, lens_host: *const i32, next_host: *mut u32) -> i32;
    pub fn rb_model_generate_step(m: *mut rb_model, tokens_host: *const u32, batch: i32, seq: i32, pos: i32, next_host: *mut u32) -> i32;
    pub fn rb_model_decode_loop(m: *mut rb_model, tokens_dev: *const u32, batch: i32, pos: i32, steps: i32, out_dev: *mut u32) -> i32;
    pub fn rb_model_set_sampling(m: *mut rb_model, repeat_penalty: f32, repeat_last_n: i32, eos_token: i32) -> i32;
    pub fn rb_model_finished(m: *mut rb_model, batch: i32, flags_host: *mut u8) -> i32;
    pub fn rb_model_decode_graph_active(m: *mut rb_model) -> i32;
    pub fn rb_model_clear_kv_cache(m: *mut rb_model) -> i32;
    pub fn rb_model_kv_cache(m: *mut rb_model) -> *mut rb_kv_cache;
    pub fn rb_launch_count(ctx: *mut rb_ctx) -> i64;
    pub fn rb_profile_start(ctx: *mut rb_ctx) -> i32;
    pub fn rb_profile_read(ctx: *mut rb_ctx, kernel_class: i32, out4: *mut f64) -> i32;
    pub fn rb_model_param_bytes(m: *mut rb_model) -> i64;
}
// </ffi>

// Tags of include/rai_b200.h (same order as rai-core/src/dtype.rs:198-524).
pub const RB_U8: i32 = 0;
pub const RB_U32: i32 = 1;
pub const RB_I64: i32 = 2;
pub const RB_F16: i32 = 3;
pub const RB_BF16: i32 = 4;
pub const RB_F32: i32 = 5;
pub const RB_F64: i32 = 6;
const UN_NEG: i32 = 0;
const UN_EXP: i32 = 1;
const UN_SQRT: i32 = 2;
const UN_RSQRT: i32 = 3;
const UN_SQUARE: i32 = 4;
const UN_TANH: i32 = 5;
const UN_ERF: i32 = 6;
const UN_SIN: i32 = 7;
const UN_COS: i32 = 8;
const UN_POWF: i32 = 9;
const UN_LOG: i32 = 14;
const UN_ABS: i32 = 15;
const UN_SIGN: i32 = 19;
const UN_LOG2: i32 = 20;
const UN_LOG10: i32 = 21;
const CMP_EQ: i32 = 0;
const CMP_NE: i32 = 1;
const CMP_GT: i32 = 2;
const CMP_GE: i32 = 3;
const CMP_LT: i32 = 4;
const CMP_LE: i32 = 5;
const BIN_ADD: i32 = 0;
const BIN_SUB: i32 = 1;
const BIN_MUL: i32 = 2;
const BIN_DIV: i32 = 3;
const BIN_MAXIMUM: i32 = 4;
const BIN_MINIMUM: i32 = 5;
const RED_SUM: i32 = 0;
const RED_MAX: i32 = 1;
const RED_MIN: i32 = 2;

#[inline]
fn check(status: i32) {
    if status != 0 {
        let msg = unsafe { CStr::from_ptr(rb_last_error()) }.to_string_lossy().into_owned();
        panic!("rai_b200 error {status}: {msg}");
    }
}

// ------------------------------------------------------------------------------------------------ contexts
/// One library context per CUDA device id, created on first use (the counterpart of the device cache at
/// candle.rs:141-175).  The pointer is stored as usize so that the map is Send + Sync; a context is only ever used
/// from the thread that evaluates the graph (rai's graph is Rc-based and single-threaded).
static CONTEXTS: Lazy<RwLock<HashMap<usize, usize>>> = Lazy::new(|| RwLock::new(HashMap::new()));

fn ctx_of(dev: &Cuda) -> *mut rb_ctx {
    if let Some(c) = CONTEXTS.read().unwrap().get(&dev.id()) {
        return *c as *mut rb_ctx;
    }
    let mut map = CONTEXTS.write().unwrap();
    let entry = map.entry(dev.id()).or_insert_with(|| {
        let mut c: *mut rb_ctx = std::ptr::null_mut();
        check(unsafe { rb_init(dev.id() as i32, &mut c) });
        c as usize
    });
    *entry as *mut rb_ctx
}

// ------------------------------------------------------------------------------------------------ storage
struct Allocation {
    ptr: *mut c_void,
    ctx: *mut rb_ctx,
}
impl Drop for Allocation {
    fn drop(&mut self) {
        // stream-ordered: kernels already enqueued on the context's stream still see the memory
        unsafe { rb_free_async(self.ctx, self.ptr) };
    }
}

/// A (possibly strided) view of a device buffer.  Strides and the offset are in elements.
#[derive(Clone)]
pub struct B200Tensor {
    buf: Rc<Allocation>,
    offset: usize,
    shape: Vec<usize>,
    strides: Vec<usize>,
    dtype: Box<dyn DType>,
}

fn dense_strides(shape: &[usize]) -> Vec<usize> {
    let mut s = vec![1usize; shape.len()];
    for i in (0..shape.len().saturating_sub(1)).rev() {
        s[i] = s[i + 1] * shape[i + 1];
    }
    s
}

fn tag(dtype: &dyn DType) -> i32 {
    let id = dtype.as_any().type_id();
    if id == TypeId::of::<U8>() {
        RB_U8
    } else if id == TypeId::of::<U32>() {
        RB_U32
    } else if id == TypeId::of::<I64>() {
        RB_I64
    } else if id == TypeId::of::<F16>() {
        RB_F16
    } else if id == TypeId::of::<BF16>() {
        RB_BF16
    } else if id == TypeId::of::<F32>() {
        RB_F32
    } else if id == TypeId::of::<F64>() {
        RB_F64
    } else {
        panic!("rai_b200: dtype {dtype:?} has no tag")
    }
}

fn elem_size(t: i32) -> usize {
    match t {
        RB_U8 => 1,
        RB_F16 | RB_BF16 => 2,
        RB_U32 | RB_F32 => 4,
        _ => 8,
    }
}

impl B200Tensor {
    fn alloc(ctx: *mut rb_ctx, shape: &[usize], dtype: &dyn DType) -> Self {
        let n: usize = shape.iter().product();
        let mut p: *mut c_void = std::ptr::null_mut();
        check(unsafe { rb_malloc_async(ctx, n.max(1) * elem_size(tag(dtype)), &mut p) });
        B200Tensor {
            buf: Rc::new(Allocation { ptr: p, ctx }),
            offset: 0,
            shape: shape.to_vec(),
            strides: dense_strides(shape),
            dtype: dtype.clone_boxed(),
        }
    }
    fn ctx(&self) -> *mut rb_ctx {
        self.buf.ctx
    }
    fn numel(&self) -> usize {
        self.shape.iter().product()
    }
    fn es(&self) -> usize {
        elem_size(tag(self.dtype.as_ref()))
    }
    fn ptr(&self) -> *mut c_void {
        unsafe { (self.buf.ptr as *mut u8).add(self.offset * self.es()) as *mut c_void }
    }
    fn is_dense(&self) -> bool {
        self.strides == dense_strides(&self.shape)
    }
    fn view(&self, offset: usize, shape: Vec<usize>, strides: Vec<usize>) -> Self {
        B200Tensor { buf: self.buf.clone(), offset, shape, strides, dtype: self.dtype.clone_boxed() }
    }
    /// A dense tensor with the same contents (self when it already is one): ToContiguous, candle.rs:980-988.
    fn dense(&self) -> Self {
        if self.is_dense() {
            return self.clone();
        }
        let out = B200Tensor::alloc(self.ctx(), &self.shape, self.dtype.as_ref());
        let shape: Vec<i64> = self.shape.iter().map(|&d| d as i64).collect();
        let xs: Vec<i64> = self.strides.iter().map(|&d| d as i64).collect();
        let os: Vec<i64> = out.strides.iter().map(|&d| d as i64).collect();
        check(unsafe {
            rb_copy_strided(self.ctx(), self.buf.ptr, xs.as_ptr(), self.offset as i64, out.buf.ptr, os.as_ptr(), 0,
                            shape.len() as i32, shape.as_ptr(), self.es() as i32)
        });
        out
    }
    fn download(&self) -> Vec<u8> {
        let d = self.dense();
        let mut v = vec![0u8; d.numel() * d.es()];
        check(unsafe { rb_download(d.ctx(), v.as_mut_ptr() as *mut c_void, d.ptr(), v.len()) });
        v
    }
}

impl fmt::Debug for B200Tensor {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        write!(f, "B200Tensor(shape={:?}, strides={:?}, dtype={:?})", self.shape, self.strides, self.dtype)
    }
}
impl fmt::Display for B200Tensor {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        fmt::Debug::fmt(self, f)
    }
}

fn typed<T: Copy>(bytes: &[u8]) -> Vec<T> {
    let n = bytes.len() / std::mem::size_of::<T>();
    let mut v = Vec::<T>::with_capacity(n);
    unsafe {
        std::ptr::copy_nonoverlapping(bytes.as_ptr(), v.as_mut_ptr() as *mut u8, n * std::mem::size_of::<T>());
        v.set_len(n);
    }
    v
}

impl TensorLike for B200Tensor {
    fn as_any(&self) -> &dyn Any {
        self
    }
    fn shape(&self) -> &[usize] {
        &self.shape
    }
    fn dtype(&self) -> &dyn DType {
        self.dtype.as_ref()
    }
    // as candle.rs:40-63: a boxed Vec / scalar of the dtype's Repr
    fn as_vec(&self) -> Box<dyn Any> {
        let b = self.download();
        match tag(self.dtype.as_ref()) {
            RB_U8 => Box::new(b),
            RB_U32 => Box::new(typed::<u32>(&b)),
            RB_I64 => Box::new(typed::<i64>(&b)),
            RB_F16 => Box::new(typed::<f16>(&b)),
            RB_BF16 => Box::new(typed::<bf16>(&b)),
            RB_F32 => Box::new(typed::<f32>(&b)),
            _ => Box::new(typed::<f64>(&b)),
        }
    }
    fn as_scalar(&self) -> Box<dyn Any> {
        assert_eq!(self.numel(), 1, "as_scalar on a tensor of {} elements", self.numel());
        let b = self.download();
        match tag(self.dtype.as_ref()) {
            RB_U8 => Box::new(b[0]),
            RB_U32 => Box::new(typed::<u32>(&b)[0]),
            RB_I64 => Box::new(typed::<i64>(&b)[0]),
            RB_F16 => Box::new(typed::<f16>(&b)[0]),
            RB_BF16 => Box::new(typed::<bf16>(&b)[0]),
            RB_F32 => Box::new(typed::<f32>(&b)[0]),
            _ => Box::new(typed::<f64>(&b)[0]),
        }
    }
    fn as_bytes(&self) -> Vec<u8> {
        self.download()
    }
}

// ------------------------------------------------------------------------------------------------ backend
#[derive(Debug, Clone, Copy, Default, PartialEq, Eq)]
pub struct B200Backend;

impl Backend for B200Backend {
    fn clone_boxed(&self) -> Box<dyn Backend> {
        Box::new(*self)
    }
    fn data_type_id(&self) -> TypeId {
        TypeId::of::<B200Tensor>()
    }
    fn as_any(&self) -> &dyn Any {
        self
    }
    fn equal(&self, rhs: &dyn Backend) -> bool {
        rhs.as_any().downcast_ref::<Self>().map_or(false, |o| o == self)
    }
}

type Data = B200Tensor;

#[inline]
fn data(t: &Tensor) -> impl Deref<Target = Data> + '_ {
    t.get_data::<Data>().expect("input is evaluated on the B200 backend")
}

// ------------------------------------------------------------------------------------------------ creation
// Full<D> (candle.rs:197-209), Arange<D> (241-273), FromArray<D> (211-239)
impl<T: Type> Eval<Cuda, ops::Full<T>> for B200Backend
where
    T::Repr: Into<f64> + Copy,
{
    fn eval(&self, dev: &Cuda, op: &ops::Full<T>, _: &[Tensor], output: &Tensor) {
        let out = B200Tensor::alloc(ctx_of(dev), output.shape(), output.dtype());
        check(unsafe { rb_fill(out.ctx(), out.ptr(), out.numel() as i64, op.val.into(), tag(output.dtype())) });
        output.set_data(out);
    }
}

impl<T: Type> Eval<Cuda, ops::Arange<T>> for B200Backend
where
    T::Repr: Into<f64> + Copy,
{
    fn eval(&self, dev: &Cuda, op: &ops::Arange<T>, _: &[Tensor], output: &Tensor) {
        let out = B200Tensor::alloc(ctx_of(dev), output.shape(), output.dtype());
        check(unsafe {
            rb_arange(out.ctx(), out.ptr(), out.numel() as i64, op.start.into(), op.step.into(), tag(output.dtype()))
        });
        output.set_data(out);
    }
}

impl<T: Type> Eval<Cuda, ops::FromArray<T>> for B200Backend {
    fn eval(&self, dev: &Cuda, op: &ops::FromArray<T>, _: &[Tensor], output: &Tensor) {
        let out = B200Tensor::alloc(ctx_of(dev), output.shape(), output.dtype());
        let bytes = op.data.len() * std::mem::size_of::<T::Repr>();
        check(unsafe { rb_upload(out.ctx(), out.ptr(), op.data.as_ptr() as *const c_void, bytes) });
        check(unsafe { rb_sync(out.ctx()) }); // `op.data` may be dropped with the node right after
        output.set_data(out);
    }
}

// ------------------------------------------------------------------------------------------------ device moves
// ToDevice<Cuda> evaluated on Cpu data (upload) and ToDevice<Cpu> evaluated on Cuda data (download); the reference
// registers both only with its `cuda` feature (dispatch.rs:117-121, rule at candle.rs:776-790).  The Cpu side's
// storage stays the reference's (`candle_core::Tensor`), so the Cpu path is untouched.
impl Eval<Cpu, ops::ToDevice<Cuda>> for B200Backend {
    fn eval(&self, _: &Cpu, op: &ops::ToDevice<Cuda>, inputs: &[Tensor], output: &Tensor) {
        let x = &inputs[0];
        let host = x.get_data::<candle_core::Tensor>().expect("Cpu storage");
        let bytes = TensorLike::as_bytes(host.deref());
        let out = B200Tensor::alloc(ctx_of(&op.device), output.shape(), output.dtype());
        check(unsafe { rb_upload(out.ctx(), out.ptr(), bytes.as_ptr() as *const c_void, bytes.len()) });
        check(unsafe { rb_sync(out.ctx()) });
        output.set_data(out);
    }
}

impl Eval<Cuda, ops::ToDevice<Cpu>> for B200Backend {
    fn eval(&self, _: &Cuda, _: &ops::ToDevice<Cpu>, inputs: &[Tensor], output: &Tensor) {
        let x = data(&inputs[0]);
        let bytes = x.download();
        let dt = match tag(x.dtype.as_ref()) {
            RB_U8 => candle_core::DType::U8,
            RB_U32 => candle_core::DType::U32,
            RB_I64 => candle_core::DType::I64,
            RB_F16 => candle_core::DType::F16,
            RB_BF16 => candle_core::DType::BF16,
            RB_F32 => candle_core::DType::F32,
            _ => candle_core::DType::F64,
        };
        let t = candle_core::Tensor::from_raw_buffer(&bytes, dt, output.shape(), &candle_core::Device::Cpu).unwrap();
        output.set_data(t);
    }
}

impl Eval<Cuda, ops::ToDevice<Cuda>> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::ToDevice<Cuda>, inputs: &[Tensor], output: &Tensor) {
        // same device: share the buffer; another GPU: through the host (peer copies are the tensor-parallel
        // driver's business, not the graph's)
        let x = data(&inputs[0]);
        if ctx_of(&op.device) == x.ctx() {
            output.set_data(x.clone());
        } else {
            let bytes = x.download();
            let out = B200Tensor::alloc(ctx_of(&op.device), output.shape(), output.dtype());
            check(unsafe { rb_upload(out.ctx(), out.ptr(), bytes.as_ptr() as *const c_void, bytes.len()) });
            check(unsafe { rb_sync(out.ctx()) });
            output.set_data(out);
        }
    }
}

// ------------------------------------------------------------------------------------------------ elementwise
// Unary rules (candle.rs:445-473,525-553,618-626,947-978): one kernel over the dense input.
macro_rules! unary_rule {
    ($op:ty, $tag:expr) => {
        impl Eval<Cuda, $op> for B200Backend {
            fn eval(&self, _: &Cuda, _: &$op, inputs: &[Tensor], output: &Tensor) {
                let x = data(&inputs[0]).dense();
                let out = B200Tensor::alloc(x.ctx(), &x.shape, x.dtype.as_ref());
                check(unsafe { rb_unary(x.ctx(), $tag, x.ptr(), out.ptr(), x.numel() as i64, 0.0, tag(x.dtype.as_ref())) });
                output.set_data(out);
            }
        }
    };
}
unary_rule!(ops::Negative, UN_NEG);
unary_rule!(ops::Exp, UN_EXP);
unary_rule!(ops::Sqrt, UN_SQRT);
unary_rule!(ops::Rsqrt, UN_RSQRT);
unary_rule!(ops::Square, UN_SQUARE);
unary_rule!(ops::Tanh, UN_TANH);
unary_rule!(ops::Erf, UN_ERF);
unary_rule!(ops::Sin, UN_SIN);
unary_rule!(ops::Cos, UN_COS);
unary_rule!(ops::Log, UN_LOG);
unary_rule!(ops::Abs, UN_ABS);
unary_rule!(ops::Sign, UN_SIGN);
unary_rule!(ops::Log2, UN_LOG2);
unary_rule!(ops::Log10, UN_LOG10);

impl<T: Type> Eval<Cuda, ops::Powf<T>> for B200Backend
where
    T::Repr: crate::FloatElemType + Into<f64> + Copy,
{
    fn eval(&self, _: &Cuda, op: &ops::Powf<T>, inputs: &[Tensor], output: &Tensor) {
        let x = data(&inputs[0]).dense();
        let out = B200Tensor::alloc(x.ctx(), &x.shape, x.dtype.as_ref());
        let e: f64 = op.exponent.into();
        check(unsafe { rb_unary(x.ctx(), UN_POWF, x.ptr(), out.ptr(), x.numel() as i64, e as f32, tag(x.dtype.as_ref())) });
        output.set_data(out);
    }
}

// Binary rules (candle.rs:275-325).  rai inserts explicit Broadcast nodes before a binary op, and Broadcast below
// is a stride-0 view, so the operands arrive with equal shapes and possibly zero strides: rb_binary takes strides.
macro_rules! binary_rule {
    ($op:ty, $tag:expr) => {
        impl Eval<Cuda, $op> for B200Backend {
            fn eval(&self, _: &Cuda, _: &$op, inputs: &[Tensor], output: &Tensor) {
                let (a, b) = (data(&inputs[0]), data(&inputs[1]));
                assert!(a.shape.len() <= 4, "rb_binary takes up to 4 dimensions; flatten leading ones first");
                let out = B200Tensor::alloc(a.ctx(), output.shape(), output.dtype());
                let shape: Vec<i64> = a.shape.iter().map(|&d| d as i64).collect();
                let sa: Vec<i64> = a.strides.iter().map(|&d| d as i64).collect();
                let sb: Vec<i64> = b.strides.iter().map(|&d| d as i64).collect();
                check(unsafe {
                    rb_binary(a.ctx(), $tag, a.ptr(), sa.as_ptr(), b.ptr(), sb.as_ptr(), out.ptr(), shape.len() as i32,
                              shape.as_ptr(), tag(a.dtype.as_ref()))
                });
                output.set_data(out);
            }
        }
    };
}
binary_rule!(ops::Add, BIN_ADD);
binary_rule!(ops::Sub, BIN_SUB);
binary_rule!(ops::Mul, BIN_MUL);
binary_rule!(ops::Div, BIN_DIV);
binary_rule!(ops::Maximum, BIN_MAXIMUM);
binary_rule!(ops::Minimum, BIN_MINIMUM);

// Comparisons (candle.rs:628-752): U8 results, operands as the binary rules take them.
macro_rules! compare_rule {
    ($op:ty, $tag:expr) => {
        impl Eval<Cuda, $op> for B200Backend {
            fn eval(&self, _: &Cuda, _: &$op, inputs: &[Tensor], output: &Tensor) {
                let (a, b) = (data(&inputs[0]), data(&inputs[1]));
                assert!(a.shape.len() <= 4, "rb_compare takes up to 4 dimensions; flatten leading ones first");
                let out = B200Tensor::alloc(a.ctx(), output.shape(), output.dtype());
                let shape: Vec<i64> = a.shape.iter().map(|&d| d as i64).collect();
                let sa: Vec<i64> = a.strides.iter().map(|&d| d as i64).collect();
                let sb: Vec<i64> = b.strides.iter().map(|&d| d as i64).collect();
                check(unsafe {
                    rb_compare(a.ctx(), $tag, a.ptr(), sa.as_ptr(), b.ptr(), sb.as_ptr(), out.ptr() as *mut u8,
                               shape.len() as i32, shape.as_ptr(), tag(a.dtype.as_ref()))
                });
                output.set_data(out);
            }
        }
    };
}
compare_rule!(ops::Equal, CMP_EQ);
compare_rule!(ops::NotEqual, CMP_NE);
compare_rule!(ops::Greater, CMP_GT);
compare_rule!(ops::GreaterEqual, CMP_GE);
compare_rule!(ops::Less, CMP_LT);
compare_rule!(ops::LessEqual, CMP_LE);

impl<T: Type> Eval<Cuda, ops::ToDType<T>> for B200Backend {
    fn eval(&self, _: &Cuda, _: &ops::ToDType<T>, inputs: &[Tensor], output: &Tensor) {
        let x = data(&inputs[0]).dense();
        let out = B200Tensor::alloc(x.ctx(), &x.shape, output.dtype());
        check(unsafe { rb_cast(x.ctx(), x.ptr(), tag(x.dtype.as_ref()), out.ptr(), tag(output.dtype()), x.numel() as i64) });
        output.set_data(out);
    }
}

// Where: inputs are [on_true, on_false, cond] (ops/where.rs:42-43, candle.rs:901-915); cond is U8.
impl Eval<Cuda, ops::Where> for B200Backend {
    fn eval(&self, _: &Cuda, _: &ops::Where, inputs: &[Tensor], output: &Tensor) {
        let (t, f, c) = (data(&inputs[0]).dense(), data(&inputs[1]).dense(), data(&inputs[2]).dense());
        let out = B200Tensor::alloc(t.ctx(), &t.shape, t.dtype.as_ref());
        check(unsafe {
            rb_where(t.ctx(), c.ptr() as *const u8, t.ptr(), f.ptr(), out.ptr(), t.numel() as i64, tag(t.dtype.as_ref()))
        });
        output.set_data(out);
    }
}

// ------------------------------------------------------------------------------------------------ contractions
// MatMul (candle.rs:401-443): [.., m, k] x [.., k, n].  Linear::fwd broadcasts W to [B, out, in] and transposes it
// (linear.rs:59-69): that arrives here as a view whose batch stride is 0 and whose last two strides are swapped,
// which is exactly rb_matmul's trans_b = 1 with b_batch_stride = 0 — ONE GEMM of M = B*S rows instead of B of them.
impl Eval<Cuda, ops::MatMul> for B200Backend {
    fn eval(&self, _: &Cuda, _: &ops::MatMul, inputs: &[Tensor], output: &Tensor) {
        let a = data(&inputs[0]).dense();
        let b = data(&inputs[1]);
        let r = a.shape.len();
        let (m, k) = (a.shape[r - 2], a.shape[r - 1]);
        let n = *b.shape.last().unwrap();
        let batch: usize = a.shape[..r - 2].iter().product();
        let rb = b.shape.len();
        // is B a transposed view of a dense [n, k] matrix, possibly broadcast over the batch?
        let transposed = b.strides[rb - 1] == k && b.strides[rb - 2] == 1;
        let bcast = b.strides[..rb - 2].iter().all(|&s| s == 0);
        let out = B200Tensor::alloc(a.ctx(), output.shape(), output.dtype());
        if transposed && (bcast || batch == 1) {
            // all batch entries share one weight: fold the batch into M
            check(unsafe {
                rb_matmul(a.ctx(), a.ptr(), b.ptr(), out.ptr(), 1, (batch * m) as i64, n as i64, k as i64, 0, 0, 1,
                          tag(a.dtype.as_ref()))
            });
        } else {
            let bd = b.dense();
            check(unsafe {
                rb_matmul(a.ctx(), a.ptr(), bd.ptr(), out.ptr(), batch as i64, m as i64, n as i64, k as i64, (m * k) as i64,
                          (k * n) as i64, 0, tag(a.dtype.as_ref()))
            });
        }
        output.set_data(out);
    }
}

// Softmax over any dim (candle.rs:792-826): rows are formed by moving `dim` last.
impl Eval<Cuda, ops::Softmax> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::Softmax, inputs: &[Tensor], output: &Tensor) {
        let x = data(&inputs[0]);
        let last = x.shape.len() - 1;
        let moved = if op.dim == last { x.dense() } else { transpose_view(&x, op.dim, last).dense() };
        let cols = *moved.shape.last().unwrap();
        let rows = moved.numel() / cols;
        let y = B200Tensor::alloc(x.ctx(), &moved.shape, x.dtype.as_ref());
        check(unsafe { rb_softmax_rows(x.ctx(), moved.ptr(), y.ptr(), rows as i64, cols as i64, tag(x.dtype.as_ref())) });
        output.set_data(if op.dim == last { y } else { transpose_view(&y, op.dim, last).dense() });
    }
}

// LogSoftmax (candle.rs:805-826), the same row layout as Softmax.
impl Eval<Cuda, ops::LogSoftmax> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::LogSoftmax, inputs: &[Tensor], output: &Tensor) {
        let x = data(&inputs[0]);
        let last = x.shape.len() - 1;
        let moved = if op.dim == last { x.dense() } else { transpose_view(&x, op.dim, last).dense() };
        let cols = *moved.shape.last().unwrap();
        let rows = moved.numel() / cols;
        let y = B200Tensor::alloc(x.ctx(), &moved.shape, x.dtype.as_ref());
        check(unsafe { rb_log_softmax_rows(x.ctx(), moved.ptr(), y.ptr(), rows as i64, cols as i64, tag(x.dtype.as_ref())) });
        output.set_data(if op.dim == last { y } else { transpose_view(&y, op.dim, last).dense() });
    }
}

// ReduceSum / ReduceMax / ReduceMin over any set of dims (ops/reduce_sum.rs:63-76, candle.rs:475-523): the reduced
// dims are permuted to the end and flattened, then one row reduction.
fn reduce(x: &B200Tensor, dims: &[usize], keep_dim: bool, kind: i32, out_shape: &[usize]) -> B200Tensor {
    let rank = x.shape.len();
    let kept: Vec<usize> = (0..rank).filter(|d| !dims.contains(d)).collect();
    let mut perm = kept.clone();
    perm.extend_from_slice(dims);
    let moved = permute_view(x, &perm).dense();
    let cols: usize = dims.iter().map(|&d| x.shape[d]).product();
    let rows = moved.numel() / cols.max(1);
    let mut out = B200Tensor::alloc(x.ctx(), out_shape, x.dtype.as_ref());
    check(unsafe { rb_reduce_rows(x.ctx(), kind, moved.ptr(), out.ptr(), rows as i64, cols as i64, tag(x.dtype.as_ref())) });
    let _ = keep_dim; // the node's shape (with or without the reduced dims as 1s) is `out_shape` either way
    out.strides = dense_strides(out_shape);
    out
}
macro_rules! reduce_rule {
    ($op:ty, $kind:expr) => {
        impl Eval<Cuda, $op> for B200Backend {
            fn eval(&self, _: &Cuda, op: &$op, inputs: &[Tensor], output: &Tensor) {
                let x = data(&inputs[0]);
                output.set_data(reduce(&x, &op.dims, op.keep_dim, $kind, output.shape()));
            }
        }
    };
}
reduce_rule!(ops::ReduceSum, RED_SUM);
reduce_rule!(ops::ReduceMax, RED_MAX);
reduce_rule!(ops::ReduceMin, RED_MIN);

// ArgMax (candle.rs:917-931): U32 indices; last index among equal maxima, like the examples' host sampler.
impl Eval<Cuda, ops::ArgMax> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::ArgMax, inputs: &[Tensor], output: &Tensor) {
        let x = data(&inputs[0]);
        let last = x.shape.len() - 1;
        let moved = if op.dim == last { x.dense() } else { transpose_view(&x, op.dim, last).dense() };
        let cols = *moved.shape.last().unwrap();
        let rows = moved.numel() / cols;
        let out = B200Tensor::alloc(x.ctx(), output.shape(), output.dtype());
        check(unsafe {
            rb_argmax_rows(x.ctx(), moved.ptr(), tag(x.dtype.as_ref()), rows as i64, cols as i64, out.ptr() as *mut u32)
        });
        output.set_data(out);
    }
}

// ArgMin (candle.rs:933-945): as ArgMax.
impl Eval<Cuda, ops::ArgMin> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::ArgMin, inputs: &[Tensor], output: &Tensor) {
        let x = data(&inputs[0]);
        let last = x.shape.len() - 1;
        let moved = if op.dim == last { x.dense() } else { transpose_view(&x, op.dim, last).dense() };
        let cols = *moved.shape.last().unwrap();
        let rows = moved.numel() / cols;
        let out = B200Tensor::alloc(x.ctx(), output.shape(), output.dtype());
        check(unsafe {
            rb_argmin_rows(x.ctx(), moved.ptr(), tag(x.dtype.as_ref()), rows as i64, cols as i64, out.ptr() as *mut u32)
        });
        output.set_data(out);
    }
}

// ------------------------------------------------------------------------------------------------ indexing
// IndexSelect (candle.rs:867-878): x viewed as [outer, dim, inner]; bit-exact row copies.
impl Eval<Cuda, ops::IndexSelect> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::IndexSelect, inputs: &[Tensor], output: &Tensor) {
        let (x, idx) = (data(&inputs[0]).dense(), data(&inputs[1]).dense());
        let outer: usize = x.shape[..op.dim].iter().product();
        let inner: usize = x.shape[op.dim + 1..].iter().product();
        let out = B200Tensor::alloc(x.ctx(), output.shape(), output.dtype());
        check(unsafe {
            rb_index_select(x.ctx(), x.ptr(), outer as i64, x.shape[op.dim] as i64, inner as i64, idx.ptr() as *const u32,
                            idx.numel() as i64, out.ptr(), x.es() as i32)
        });
        output.set_data(out);
    }
}

// Gather (candle.rs:838-849) along the last dim; other dims are moved last first.
impl Eval<Cuda, ops::Gather> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::Gather, inputs: &[Tensor], output: &Tensor) {
        let (x, idx) = (data(&inputs[0]), data(&inputs[1]));
        let last = x.shape.len() - 1;
        let (xm, im) = if op.dim == last {
            (x.dense(), idx.dense())
        } else {
            (transpose_view(&x, op.dim, last).dense(), transpose_view(&idx, op.dim, last).dense())
        };
        let cols = *xm.shape.last().unwrap();
        let k = *im.shape.last().unwrap();
        let rows = xm.numel() / cols;
        let y = B200Tensor::alloc(x.ctx(), &im.shape, x.dtype.as_ref());
        check(unsafe {
            rb_gather_last(x.ctx(), xm.ptr(), rows as i64, cols as i64, im.ptr() as *const u32, k as i64, y.ptr(), x.es() as i32)
        });
        output.set_data(if op.dim == last { y } else { transpose_view(&y, op.dim, last).dense() });
    }
}

// ScatterAdd / IndexAdd (candle.rs:851-865, 991-1004): inputs are [x, source, index]; x viewed as [outer, dim, inner].
// ScatterAdd's index has the source's shape, IndexAdd's is one-dimensional along `dim`.
fn scatter(x: &B200Tensor, src: &B200Tensor, idx: &B200Tensor, dim: usize, index_is_1d: bool, output: &Tensor) {
    let (x, src, idx) = (x.dense(), src.dense(), idx.dense());
    let outer: usize = x.shape[..dim].iter().product();
    let inner: usize = x.shape[dim + 1..].iter().product();
    let out = B200Tensor::alloc(x.ctx(), output.shape(), output.dtype());
    check(unsafe {
        rb_scatter_add(x.ctx(), x.ptr(), src.ptr(), idx.ptr() as *const u32, out.ptr(), outer as i64, x.shape[dim] as i64,
                       src.shape[dim] as i64, inner as i64, index_is_1d as i32, tag(x.dtype.as_ref()))
    });
    output.set_data(out);
}
impl Eval<Cuda, ops::ScatterAdd> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::ScatterAdd, inputs: &[Tensor], output: &Tensor) {
        scatter(&data(&inputs[0]), &data(&inputs[1]), &data(&inputs[2]), op.dim, false, output);
    }
}
impl Eval<Cuda, ops::IndexAdd> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::IndexAdd, inputs: &[Tensor], output: &Tensor) {
        scatter(&data(&inputs[0]), &data(&inputs[1]), &data(&inputs[2]), op.dim, true, output);
    }
}

// ------------------------------------------------------------------------------------------------ convolutions, pools
// NCHW activations, [out, in, kh, kw] weights ([in, out, kh, kw] transposed), as candle.rs:1006-1150 passes them on.
// The 1-D forms run as the 2-D ones over a height of one.
fn i32x4(shape: &[usize]) -> [i32; 4] {
    [shape[0] as i32, shape[1] as i32, shape[2] as i32, shape[3] as i32]
}
fn with_unit_height(x: &B200Tensor) -> B200Tensor {
    let d = x.dense();
    let shape = vec![d.shape[0], d.shape[1], 1, d.shape[2]];
    let strides = dense_strides(&shape);
    d.view(d.offset, shape, strides)
}
fn conv2d(x: &B200Tensor, w: &B200Tensor, padding: [i32; 2], stride: [i32; 2], dilation: [i32; 2], output: &Tensor) {
    let (x, w) = (x.dense(), w.dense());
    let mut oshape = [0i32; 4];
    let out = B200Tensor::alloc(x.ctx(), output.shape(), output.dtype());
    check(unsafe {
        rb_conv2d(x.ctx(), x.ptr(), i32x4(&x.shape).as_ptr(), w.ptr(), i32x4(&w.shape).as_ptr(), padding.as_ptr(),
                  stride.as_ptr(), dilation.as_ptr(), out.ptr(), oshape.as_mut_ptr(), tag(x.dtype.as_ref()))
    });
    output.set_data(out);   // the node's own shape ([N, C, L] for the 1-D form) over the same dense bytes
}
impl Eval<Cuda, ops::Conv2d> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::Conv2d, inputs: &[Tensor], output: &Tensor) {
        let p = |a: [usize; 2]| [a[0] as i32, a[1] as i32];
        conv2d(&data(&inputs[0]), &data(&inputs[1]), p(op.padding), p(op.stride), p(op.dilation), output);
    }
}
impl Eval<Cuda, ops::Conv1d> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::Conv1d, inputs: &[Tensor], output: &Tensor) {
        conv2d(&with_unit_height(&data(&inputs[0])), &with_unit_height(&data(&inputs[1])), [0, op.padding as i32],
               [1, op.stride as i32], [1, op.dilation as i32], output);
    }
}
fn conv_transpose2d(x: &B200Tensor, w: &B200Tensor, padding: [i32; 2], out_padding: [i32; 2], stride: [i32; 2],
                    dilation: [i32; 2], output: &Tensor) {
    let (x, w) = (x.dense(), w.dense());
    let mut oshape = [0i32; 4];
    let out = B200Tensor::alloc(x.ctx(), output.shape(), output.dtype());
    check(unsafe {
        rb_conv_transpose2d(x.ctx(), x.ptr(), i32x4(&x.shape).as_ptr(), w.ptr(), i32x4(&w.shape).as_ptr(), padding.as_ptr(),
                            out_padding.as_ptr(), stride.as_ptr(), dilation.as_ptr(), out.ptr(), oshape.as_mut_ptr(),
                            tag(x.dtype.as_ref()))
    });
    output.set_data(out);
}
impl Eval<Cuda, ops::ConvTranspose2d> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::ConvTranspose2d, inputs: &[Tensor], output: &Tensor) {
        let p = |a: [usize; 2]| [a[0] as i32, a[1] as i32];
        conv_transpose2d(&data(&inputs[0]), &data(&inputs[1]), p(op.padding), p(op.out_padding), p(op.stride),
                         p(op.dilation), output);
    }
}
impl Eval<Cuda, ops::ConvTranspose1d> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::ConvTranspose1d, inputs: &[Tensor], output: &Tensor) {
        conv_transpose2d(&with_unit_height(&data(&inputs[0])), &with_unit_height(&data(&inputs[1])), [0, op.padding as i32],
                         [0, op.output_padding as i32], [1, op.stride as i32], [1, op.dilation as i32], output);
    }
}
fn pool2d(x: &B200Tensor, is_max: bool, kernel: [i32; 2], stride: [i32; 2], padding: [i32; 2], dilation: [i32; 2],
          output: &Tensor) {
    let x = x.dense();
    let mut oshape = [0i32; 4];
    let out = B200Tensor::alloc(x.ctx(), output.shape(), output.dtype());
    check(unsafe {
        rb_pool2d(x.ctx(), is_max as i32, x.ptr(), i32x4(&x.shape).as_ptr(), kernel.as_ptr(), stride.as_ptr(),
                  padding.as_ptr(), dilation.as_ptr(), out.ptr(), oshape.as_mut_ptr(), tag(x.dtype.as_ref()))
    });
    output.set_data(out);
}
impl Eval<Cuda, ops::MaxPool2d> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::MaxPool2d, inputs: &[Tensor], output: &Tensor) {
        let p = |a: (usize, usize)| [a.0 as i32, a.1 as i32];
        pool2d(&data(&inputs[0]), true, p(op.kernel_size), p(op.stride), p(op.padding), p(op.dilation), output);
    }
}
impl Eval<Cuda, ops::AvgPool2d> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::AvgPool2d, inputs: &[Tensor], output: &Tensor) {
        let p = |a: (usize, usize)| [a.0 as i32, a.1 as i32];
        pool2d(&data(&inputs[0]), false, p(op.kernel_size), p(op.stride), p(op.padding), [1, 1], output);
    }
}
impl Eval<Cuda, ops::MaxPool1d> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::MaxPool1d, inputs: &[Tensor], output: &Tensor) {
        pool2d(&with_unit_height(&data(&inputs[0])), true, [1, op.kernel_size as i32], [1, op.stride as i32],
               [0, op.padding as i32], [1, op.dilation as i32], output);
    }
}
impl Eval<Cuda, ops::AvgPool1d> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::AvgPool1d, inputs: &[Tensor], output: &Tensor) {
        pool2d(&with_unit_height(&data(&inputs[0])), false, [1, op.kernel_size as i32], [1, op.stride as i32],
               [0, op.padding as i32], [1, 1], output);
    }
}
fn upsample_nearest2d(x: &B200Tensor, h: usize, w: usize, output: &Tensor) {
    let x = x.dense();
    let out = B200Tensor::alloc(x.ctx(), output.shape(), output.dtype());
    check(unsafe {
        rb_upsample_nearest2d(x.ctx(), x.ptr(), i32x4(&x.shape).as_ptr(), h as i32, w as i32, out.ptr(), tag(x.dtype.as_ref()))
    });
    output.set_data(out);
}
impl Eval<Cuda, ops::UpsampleNearest2d> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::UpsampleNearest2d, inputs: &[Tensor], output: &Tensor) {
        upsample_nearest2d(&data(&inputs[0]), op.size.0, op.size.1, output);
    }
}
impl Eval<Cuda, ops::UpsampleNearest1d> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::UpsampleNearest1d, inputs: &[Tensor], output: &Tensor) {
        upsample_nearest2d(&with_unit_height(&data(&inputs[0])), 1, op.size, output);
    }
}

// ------------------------------------------------------------------------------------------------ views
fn transpose_view(x: &B200Tensor, d0: usize, d1: usize) -> B200Tensor {
    let (mut shape, mut strides) = (x.shape.clone(), x.strides.clone());
    shape.swap(d0, d1);
    strides.swap(d0, d1);
    x.view(x.offset, shape, strides)
}
fn permute_view(x: &B200Tensor, perm: &[usize]) -> B200Tensor {
    x.view(x.offset, perm.iter().map(|&p| x.shape[p]).collect(), perm.iter().map(|&p| x.strides[p]).collect())
}

impl Eval<Cuda, ops::Transpose> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::Transpose, inputs: &[Tensor], output: &Tensor) {
        output.set_data(transpose_view(&data(&inputs[0]), op.dim0, op.dim1));
    }
}
impl Eval<Cuda, ops::Permute> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::Permute, inputs: &[Tensor], output: &Tensor) {
        output.set_data(permute_view(&data(&inputs[0]), &op.dims));
    }
}
impl Eval<Cuda, ops::Narrow> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::Narrow, inputs: &[Tensor], output: &Tensor) {
        let x = data(&inputs[0]);
        let mut shape = x.shape.clone();
        shape[op.dim] = op.len;
        output.set_data(x.view(x.offset + op.start * x.strides[op.dim], shape, x.strides.clone()));
    }
}
impl Eval<Cuda, ops::Broadcast> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::Broadcast, inputs: &[Tensor], output: &Tensor) {
        // right-aligned; a dimension of size 1 (or a missing leading one) is repeated with stride 0 (candle.rs:575-583)
        let x = data(&inputs[0]);
        let lead = op.shape.len() - x.shape.len();
        let strides: Vec<usize> = (0..op.shape.len())
            .map(|i| if i < lead || (x.shape[i - lead] == 1 && op.shape[i] != 1) { 0 } else { x.strides[i - lead] })
            .collect();
        output.set_data(x.view(x.offset, op.shape.clone(), strides));
    }
}
impl Eval<Cuda, ops::Reshape> for B200Backend {
    fn eval(&self, _: &Cuda, op: &ops::Reshape, inputs: &[Tensor], output: &Tensor) {
        // a dense tensor is re-viewed; anything else is made dense first (candle.rs:555-573 does the same)
        let x = data(&inputs[0]).dense();
        output.set_data(x.view(x.offset, op.shape.clone(), dense_strides(&op.shape)));
    }
}
impl Eval<Cuda, ops::ToContiguous> for B200Backend {
    fn eval(&self, _: &Cuda, _: &ops::ToContiguous, inputs: &[Tensor], output: &Tensor) {
        output.set_data(data(&inputs[0]).dense());
    }
}
// Concatenate (candle.rs:880-889): each input is copied into its slice of the output.
impl Eval<Cuda, ops::Concatenate> for B200Backend {
    fn eval(&self, dev: &Cuda, op: &ops::Concatenate, inputs: &[Tensor], output: &Tensor) {
        let out = B200Tensor::alloc(ctx_of(dev), output.shape(), output.dtype());
        let mut at = 0usize;
        for t in inputs {
            let x = data(t);
            let shape: Vec<i64> = x.shape.iter().map(|&d| d as i64).collect();
            let xs: Vec<i64> = x.strides.iter().map(|&d| d as i64).collect();
            let os: Vec<i64> = out.strides.iter().map(|&d| d as i64).collect();
            check(unsafe {
                rb_copy_strided(out.ctx(), x.buf.ptr, xs.as_ptr(), x.offset as i64, out.buf.ptr, os.as_ptr(),
                                (at * out.strides[op.dim]) as i64, shape.len() as i32, shape.as_ptr(), x.es() as i32)
            });
            at += x.shape[op.dim];
        }
        output.set_data(out);
    }
}

// ------------------------------------------------------------------------------------------------ registration
/// Installs the rules above for `Cuda`, key by key like `register_backend!` (dispatch.rs:41-157).  Ops of that list
/// with no rule here stay unregistered for `Cuda` and evaluate to `Error::Unimplemented` (eval.rs:40-43): Random and
/// Normal, which nothing on the decoders' path reaches.
pub fn register_all() {
    let b = B200Backend;
    macro_rules! reg {
        ($($op:ty),* $(,)?) => { $( dispatch::register::<Cuda, $op, B200Backend>(b); )* };
    }
    reg!(
        ops::Full<U8>, ops::Full<U32>, ops::Full<BF16>, ops::Full<F16>, ops::Full<F32>, ops::Full<F64>, ops::Full<I64>,
        ops::Arange<U8>, ops::Arange<U32>, ops::Arange<BF16>, ops::Arange<F16>, ops::Arange<F32>, ops::Arange<F64>,
        ops::Arange<I64>,
        ops::FromArray<U8>, ops::FromArray<U32>, ops::FromArray<BF16>, ops::FromArray<F16>, ops::FromArray<F32>,
        ops::FromArray<F64>, ops::FromArray<I64>,
        ops::Concatenate,
        ops::Add, ops::Sub, ops::Mul, ops::Div, ops::MatMul, ops::Maximum, ops::Minimum,
        ops::Sin, ops::Cos, ops::Tanh, ops::Negative, ops::Square,
        ops::Powf<BF16>, ops::Powf<F16>, ops::Powf<F32>, ops::Powf<F64>,
        ops::Sqrt, ops::Rsqrt, ops::Abs, ops::Exp, ops::Log, ops::Erf,
        ops::ToDType<U8>, ops::ToDType<U32>, ops::ToDType<BF16>, ops::ToDType<F16>, ops::ToDType<F32>, ops::ToDType<F64>,
        ops::ToDType<I64>,
        ops::Softmax, ops::ToDevice<Cpu>, ops::ToDevice<Cuda>,
        ops::Gather, ops::IndexSelect, ops::Narrow, ops::Where,
        ops::Transpose, ops::Reshape, ops::Permute, ops::Broadcast, ops::ToContiguous,
        ops::ReduceSum, ops::ReduceMax, ops::ReduceMin, ops::ArgMax, ops::ArgMin,
        ops::Equal, ops::NotEqual, ops::Greater, ops::GreaterEqual, ops::Less, ops::LessEqual,
        ops::Sign, ops::Log2, ops::Log10, ops::LogSoftmax, ops::ScatterAdd, ops::IndexAdd,
        ops::Conv1d, ops::Conv2d, ops::ConvTranspose1d, ops::ConvTranspose2d,
        ops::MaxPool1d, ops::MaxPool2d, ops::AvgPool1d, ops::AvgPool2d, ops::UpsampleNearest1d, ops::UpsampleNearest2d,
    );
    // the upload direction is keyed by the SOURCE device (dispatch.rs:207-212 looks rules up by the node's device)
    dispatch::register::<Cpu, ops::ToDevice<Cuda>, B200Backend>(b);
}

// ------------------------------------------------------------------------------------------------ fused decoder path
// The rules above make every node of the decoders' graphs (rai-models/src/llm/*.rs) run on the library's
// primitive kernels, about 105 launches per layer.  The fused path — 7 launches per layer, paged KV cache, captured
// decode step — is reached through the decoder driver instead, which replaces `Model::new` / `update_by_safetensors`
// / `Model::fwd` / `clear_kv_cache` of the four model files one for one:
pub struct B200Model {
    m: *mut rb_model,
    ctx: *mut rb_ctx,
    vocab: usize,
    dtype: Box<dyn DType>,
}

impl B200Model {
    /// `Model::new(cfg, dtype, device)` (qwen2.rs:287-304): `cfg` carries the fields of the model's `Config` plus the
    /// cache capacities.
    pub fn new(cfg: &rb_model_config, dev: &Cuda, dtype: &dyn DType) -> Self {
        let ctx = ctx_of(dev);
        let mut m: *mut rb_model = std::ptr::null_mut();
        check(unsafe { rb_model_create(ctx, cfg, &mut m) });
        B200Model { m, ctx, vocab: cfg.vocab_size as usize, dtype: dtype.clone_boxed() }
    }
    /// `Module::update_by_safetensors` (nn.rs:39-55).
    pub fn update_by_safetensors(&self, files: &[std::path::PathBuf]) {
        let c: Vec<std::ffi::CString> =
            files.iter().map(|p| std::ffi::CString::new(p.to_string_lossy().as_bytes()).unwrap()).collect();
        let p: Vec<*const c_char> = c.iter().map(|s| s.as_ptr()).collect();
        check(unsafe { rb_model_load_safetensors(self.m, p.as_ptr(), p.len() as i32) });
    }
    /// `Model::fwd(input, seqlen_offset)` (qwen2.rs:338-359): `input` is a U32 tensor [B, S] on this device; returns
    /// the last-position logits [B, 1, V] as a rai tensor whose storage is a `B200Tensor`.
    pub fn fwd(&self, input: &Tensor, seqlen_offset: usize) -> Tensor {
        let ids = data(input).dense();
        let (b, s) = (ids.shape[0], ids.shape[1]);
        let out = B200Tensor::alloc(self.ctx, &[b, 1, self.vocab], self.dtype.as_ref());
        check(unsafe {
            rb_model_forward(self.m, ids.ptr() as *const u32, b as i32, s as i32, seqlen_offset as i32, out.ptr())
        });
        let t = Tensor::new(input.device(), self.dtype.as_ref(), [b, 1, self.vocab], ops::ToContiguous, vec![]);
        t.set_data(out);
        t
    }
    /// `clear_kv_cache` (qwen2.rs:361-365).
    pub fn clear_kv_cache(&self) {
        check(unsafe { rb_model_clear_kv_cache(self.m) });
    }
}
impl Drop for B200Model {
    fn drop(&mut self) {
        unsafe { rb_model_destroy(self.m) };
    }
}
