//! Raw bindings of `include/ellm_attn.h` and `include/ellm_proj.h`.
//!
//! Every function returns an `ellm_status` (`0` = ok); `ellm_last_error()` holds the thread-local
//! text of the last failure.  All data pointers are DEVICE pointers unless a parameter is named
//! `*_host`.  Nothing here aborts; the reference crate is `panic = "abort"`, so its operators turn a
//! non-zero status into a panic.
#![allow(non_camel_case_types)]

use std::ffi::CStr;
use std::os::raw::{c_char, c_int, c_longlong, c_ulonglong, c_void};

pub const ELLM_OK: c_int = 0;
pub const ELLM_ERR_INVALID_ARG: c_int = 1;
pub const ELLM_ERR_CUDA: c_int = 2;
pub const ELLM_ERR_DEVICE_TIMEOUT: c_int = 3;
pub const ELLM_ERR_UNSUPPORTED: c_int = 4;
pub const ELLM_ERR_NO_MEMORY: c_int = 5;

pub const ELLM_DTYPE_BF16: c_int = 0;
pub const ELLM_PREFILL_AUTO: c_int = 0;
pub const ELLM_PREFILL_TCGEN05: c_int = 1;
pub const ELLM_PREFILL_WARP_MMA: c_int = 2;
pub const ELLM_NOALLOC_MAX_SLOTS: usize = 1024;
pub const ELLM_NOALLOC_MAX_BATCH: usize = 1024;

/// `ellm_attn_desc`: the arguments of `Attention::new` plus what a device needs.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct ellm_attn_desc {
    pub q: *const c_void,
    pub k_cache: *mut c_void,
    pub v_cache: *mut c_void,
    pub out: *mut c_void,
    pub lse: *mut f32,
    pub k_new: *const c_void,
    pub v_new: *const c_void,
    pub max_batch: usize,
    pub q_heads: usize,
    pub kv_heads: usize,
    pub head_size: usize,
    pub kv_strides: [usize; 4],
    pub max_seq: usize,
    pub max_interval: usize,
    pub scale: f32,
    pub dtype: c_int,
    pub device: c_int,
    pub stream: *mut c_void,
    pub r#async: c_int,
    pub prefill_kernel: c_int,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct ellm_matmul3_desc {
    pub hidden: *const c_void,
    pub hidden_row_stride: usize,
    pub wq_nt: *const c_void,
    pub wk_nt: *const c_void,
    pub wv_nt: *const c_void,
    pub q_state: *mut c_void,
    pub k_cache: *mut c_void,
    pub v_cache: *mut c_void,
    pub kv_strides: [usize; 4],
    pub rope: *const f32,
    pub rope_rows: usize,
    pub q_norm_weight: *const f32,
    pub k_norm_weight: *const f32,
    pub head_dim: usize,
    pub m_row: usize,
    pub col: usize,
    pub b_q_row: usize,
    pub b_kv_row: usize,
    pub max_batch: usize,
    pub max_seq: usize,
    pub eps: f32,
    pub device: c_int,
    pub stream: *mut c_void,
    pub r#async: c_int,
    pub input_norm: c_int,
    pub input_norm_eps: f32,
    pub normed_scratch: *mut c_void,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct ellm_matmul_add_desc {
    pub a: *const c_void,
    pub a_row_stride: usize,
    pub w_nt: *const c_void,
    pub residual: *const c_void,
    pub residual_row_stride: usize,
    pub output: *mut c_void,
    pub output_row_stride: usize,
    pub m_max: usize,
    pub n_max: usize,
    pub k_max: usize,
    pub max_batch: usize,
    pub device: c_int,
    pub stream: *mut c_void,
    pub r#async: c_int,
}

macro_rules! opaque {
    ($($name:ident),*) => { $( #[repr(C)] pub struct $name { _private: [u8; 0] } )* };
}
opaque!(ellm_attn, ellm_matmul3, ellm_matmul_add, ellm_kv_cache, ellm_step_graph);

#[link(name = "ellm_attn")]
extern "C" {
    // ---- the attention operator: Attention::new / run (src/compiler/mul/attention.rs:41-76)
    pub fn ellm_attn_create(desc: *const ellm_attn_desc, out: *mut *mut ellm_attn) -> c_int;
    pub fn ellm_attn_destroy(h: *mut ellm_attn) -> c_int;
    pub fn ellm_attn_run(h: *mut ellm_attn, position_index: usize, position_interval: usize,
                         batch_size: usize, cpu_num: usize, thread_id: usize) -> c_int;
    pub fn ellm_attn_run_ragged(h: *mut ellm_attn, positions: *const i32, position_interval: usize,
                                batch_size: usize, cpu_num: usize, thread_id: usize) -> c_int;
    pub fn ellm_attn_run_host(h: *mut ellm_attn, q_host: *const c_void, k_new_host: *const c_void,
                              v_new_host: *const c_void, out_host: *mut c_void, lse_host: *mut f32,
                              positions_host: *const i32, position_index: usize,
                              position_interval: usize, batch_size: usize) -> c_int;
    pub fn ellm_attn_run_window(h: *mut ellm_attn, position_index: usize, position_interval: usize,
                                batch_size: usize, key_begin: usize, key_end: usize,
                                o_part: *mut f32, lse_part: *mut f32) -> c_int;
    pub fn ellm_attn_run_window_q(h: *mut ellm_attn, q: *const c_void, position_index: usize,
                                  position_interval: usize, batch_size: usize, key_begin: usize,
                                  key_end: usize, o_part: *mut f32, lse_part: *mut f32) -> c_int;
    pub fn ellm_attn_check(h: *mut ellm_attn) -> c_int;
    pub fn ellm_attn_set_option(h: *mut ellm_attn, name: *const c_char, value: c_longlong) -> c_int;
    pub fn ellm_attn_set_profiling(h: *mut ellm_attn, on: c_int) -> c_int;
    pub fn ellm_attn_kernel_stats(h: *mut ellm_attn, kernel_id: c_int, launches: *mut u64,
                                  timed_launches: *mut u64, total_ms: *mut f64) -> c_int;
    pub fn ellm_attn_decode_noalloc(q: *const c_void, k_cache: *const c_void, v_cache: *const c_void,
                                    out: *mut c_void, lse: *mut f32, positions: *const i32,
                                    position_index: usize, batch_size: usize, q_heads: usize,
                                    kv_heads: usize, head_size: usize, kv_strides: *const usize,
                                    max_seq: usize, scale: f32, device: c_int, stream: *mut c_void) -> c_int;
    pub fn ellm_attn_merge_partials(o_parts: *const f32, lse_parts: *const f32, parts: usize, rows: usize,
                                    head_size: usize, out: *mut c_void, lse_out: *mut f32, device: c_int,
                                    stream: *mut c_void) -> c_int;
    pub fn ellm_attn_merge_partials_f32(o_parts: *const f32, lse_parts: *const f32, parts: usize, rows: usize,
                                        head_size: usize, out: *mut f32, lse_out: *mut f32, device: c_int,
                                        stream: *mut c_void) -> c_int;
    pub fn ellm_attn_merge_partials_list(o_parts: *const *const f32, lse_parts: *const *const f32, parts: usize,
                                         rows: usize, head_size: usize, out: *mut c_void, out_is_f32: c_int,
                                         lse_out: *mut f32, device: c_int, stream: *mut c_void) -> c_int;

    // ---- memory: allocate_init (src/memory/allocator.rs:16-27) and the static KV cache
    pub fn ellm_device_alloc(device: c_int, bytes: usize, out: *mut *mut c_void) -> c_int;
    pub fn ellm_device_free(device: c_int, ptr: *mut c_void) -> c_int;
    pub fn ellm_kv_cache_create(device: c_int, layers: usize, max_batch: usize, kv_heads: usize,
                                max_seq: usize, head_size: usize, out: *mut *mut ellm_kv_cache) -> c_int;
    pub fn ellm_kv_cache_destroy(cache: *mut ellm_kv_cache) -> c_int;
    pub fn ellm_kv_cache_layer(cache: *const ellm_kv_cache, layer: usize, k: *mut *mut c_void,
                               v: *mut *mut c_void, kv_strides: *mut usize) -> c_int;
    pub fn ellm_kv_append(cache: *mut c_void, src: *const c_void, kv_strides: *const usize, max_batch: usize,
                          kv_heads: usize, head_size: usize, max_seq: usize, position_index: usize,
                          positions: *const i32, position_interval: usize, batch_size: usize, device: c_int,
                          stream: *mut c_void) -> c_int;

    // ---- the steps either side of attention
    pub fn ellm_qk_norm_rope_append(q_in: *const c_void, k_in: *const c_void, v_in: *const c_void,
                                    q_out: *mut c_void, k_cache: *mut c_void, v_cache: *mut c_void,
                                    q_weight: *const f32, k_weight: *const f32, rope: *const f32,
                                    rope_rows: usize, kv_strides: *const usize, max_batch: usize,
                                    q_heads: usize, kv_heads: usize, head_size: usize, max_seq: usize,
                                    position_index: usize, positions: *const i32, position_interval: usize,
                                    batch_size: usize, eps: f32, q_in_row_stride: usize,
                                    kv_in_row_stride: usize, device: c_int, stream: *mut c_void) -> c_int;
    pub fn ellm_rms_norm(x: *const c_void, y: *mut c_void, rows: usize, length: usize, eps: f32,
                         device: c_int, stream: *mut c_void) -> c_int;
    pub fn ellm_matmul3_create(desc: *const ellm_matmul3_desc, out: *mut *mut ellm_matmul3) -> c_int;
    pub fn ellm_matmul3_destroy(h: *mut ellm_matmul3) -> c_int;
    pub fn ellm_matmul3_run(h: *mut ellm_matmul3, position_index: usize, position_interval: usize,
                            batch_size: usize, cpu_num: usize, thread_id: usize) -> c_int;
    pub fn ellm_matmul3_run_ragged(h: *mut ellm_matmul3, positions: *const i32, position_interval: usize,
                                   batch_size: usize, cpu_num: usize, thread_id: usize) -> c_int;
    pub fn ellm_matmul3_set_decode_fusion(h: *mut ellm_matmul3, on: c_int) -> c_int;
    pub fn ellm_matmul_add_create(desc: *const ellm_matmul_add_desc, out: *mut *mut ellm_matmul_add) -> c_int;
    pub fn ellm_matmul_add_destroy(h: *mut ellm_matmul_add) -> c_int;
    pub fn ellm_matmul_add_run(h: *mut ellm_matmul_add, position_index: usize, position_interval: usize,
                               batch_size: usize, cpu_num: usize, thread_id: usize) -> c_int;
    pub fn ellm_matmul_set_profiling(handle: *mut c_void, which: c_int, on: c_int) -> c_int;
    pub fn ellm_matmul_kernel_stats(handle: *mut c_void, which: c_int, launches: *mut u64,
                                    timed_launches: *mut u64, ms: *mut f64) -> c_int;
    pub fn ellm_matmul_check(handle: *mut c_void, which: c_int) -> c_int;
    pub fn ellm_matmul_set_wait_timeout(handle: *mut c_void, which: c_int, ns: c_ulonglong) -> c_int;
    pub fn ellm_matmul_set_pairing(handle: *mut c_void, which: c_int, mode: c_int) -> c_int;
    pub fn ellm_matmul_debug_skip_load(handle: *mut c_void, which: c_int, item: c_int) -> c_int;

    // ---- a step without a host barrier per operator (src/serving/start.rs:69-73 replaced)
    pub fn ellm_stream_create(device: c_int, stream: *mut *mut c_void) -> c_int;
    pub fn ellm_stream_destroy(device: c_int, stream: *mut c_void) -> c_int;
    pub fn ellm_stream_synchronize(device: c_int, stream: *mut c_void) -> c_int;
    pub fn ellm_positions_set(positions: *mut i32, count: usize, value: i32, add: c_int, device: c_int,
                              stream: *mut c_void) -> c_int;
    pub fn ellm_step_graph_begin(device: c_int, stream: *mut c_void) -> c_int;
    pub fn ellm_step_graph_end(device: c_int, stream: *mut c_void, out: *mut *mut ellm_step_graph) -> c_int;
    pub fn ellm_step_graph_launch(graph: *mut ellm_step_graph, stream: *mut c_void) -> c_int;
    pub fn ellm_step_graph_nodes(graph: *const ellm_step_graph, nodes: *mut usize) -> c_int;
    pub fn ellm_step_graph_destroy(graph: *mut ellm_step_graph) -> c_int;

    pub fn ellm_last_error() -> *const c_char;
    pub fn ellm_status_string(status: c_int) -> *const c_char;
    pub fn ellm_attn_abi_version() -> c_int;
}

/// Text of the calling thread's last failure.
pub fn last_error() -> String {
    unsafe { CStr::from_ptr(ellm_last_error()).to_string_lossy().into_owned() }
}
